// Model-loader of the decode runtime: architecture config, synthetic model
// plans, and the device-resident model (two arenas + small-weight mirrors +
// per-layer tables). Mirrors the loader section of the reference's token loop
// (tools/decode/decode_l0.cpp:127-189 parse, :228-267 arenas and staged upload,
// :296-340 small-weight mirrors, :341-354 RoPE table), with model dimensions
// read from the container's architecture section instead of compiled in.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "../../../include/ainfer_cuda.h"
#include "binfer.h"

namespace ainfer {

struct ModelConfig {
  std::string arch = "qwen3_5_moe";
  int hidden = 0, layers = 0, vocab = 0;
  std::string layer_types;  // one char per layer: 'L' Gated DeltaNet, 'A' gated GQA attention
  int q_heads = 0, kv_heads = 0, head_dim = 256, rotary_dim = 64;
  double rope_theta = 1e7;
  int lin_k_heads = 0, lin_v_heads = 0, lin_head_dim = 128, conv_kernel = 4;
  int experts = 0, top_k = 0, shared_experts = 1, expert_inter = 0;
  int mtp_layers = 0;
  double rms_eps = 1e-6;
  int conv_dim() const { return (2 * lin_k_heads + lin_v_heads) * lin_head_dim; }
  int value_dim() const { return lin_v_heads * lin_head_dim; }
  int n_attn() const { int n = 0; for (char c : layer_types) n += c == 'A'; return n; }
  int n_lin() const { int n = 0; for (char c : layer_types) n += c == 'L'; return n; }
  std::string to_json() const;
  static bool from_json(const std::string &js, ModelConfig &out, std::string &err);
  // Shapes this runtime's kernels accept; fills err with the first violation.
  bool check(std::string &err) const;
};

// Named synthetic shapes: "tiny" (CPU-test sized), "mini" (the CPU-runnable
// reference mini-model), "full" (80B-A3B-shaped). Returns false if unknown.
bool preset_config(const std::string &name, ModelConfig &out);

// How one tensor of a synthetic model is filled.
struct SynthSpec {
  float std_ = 0.02f;     // N(0, std^2) draws; 0 = constant
  float constant = 0.0f;
};
// The tensor list (names, shapes, storage) of a model of this shape, in the
// order the writer lays them out, and how each is filled when synthetic.
void build_plan(const ModelConfig &cfg, Container &c, std::vector<SynthSpec> &specs);

// Checks every tensor the decode kernels read against the architecture: presence, shape and
// storage of the projection matrices, every expert's gate/up/down, router, shared-expert gate,
// embedding and LM head. The kernels take their loop bounds from the architecture, so a
// directory that disagrees with it would make them read past the weight arenas. Host only.
// Returns 0, 1 (missing tensor) or 2 (wrong shape or storage) with the first violation in err.
int check_directory_shapes(const Container &dir, const ModelConfig &cfg, std::string &err);

// Writes a synthetic model file on the host (no GPU involved).
int synth_write_file(const char *path, const ModelConfig &cfg, uint64_t seed, std::string &err);
// SafeTensors file or directory (with model.safetensors.index.json) -> .binfer (ingest.cpp).
int binfer_from_safetensors(const char *src, const char *arch_json, const char *out_path, std::string &err);

struct DeviceTensor {
  const TensorEntry *entry = nullptr;
  void *data = nullptr;    // device address of the payload
  void *scales = nullptr;  // device address of the scales (INT4) or null
};

// Device-resident model.
struct DeviceModel {
  ainfer_device_t dev = nullptr;
  ModelConfig cfg;
  Container dir;            // directory (offsets are file offsets, or virtual ones when synthetic)
  void *pay_arena = nullptr, *sc_arena = nullptr;
  uint64_t pay_bytes = 0, sc_bytes = 0;
  uint64_t seed = 0;
  bool synthetic = false;
  std::vector<void *> owned;  // other device allocations (mirrors, tables)
  // fp32 mirrors of the small BF16 tensors, stacked per kind
  float *in_norm = nullptr, *post_norm = nullptr;       // [layers(+mtp)][H]
  float *q_norm = nullptr, *k_norm = nullptr;           // [n_attn(+mtp)][head_dim]
  float *lin_norm = nullptr;                            // [n_lin][lin_head_dim]
  float *a_log = nullptr, *dt_bias = nullptr;           // [n_lin][nV]
  float *conv_w = nullptr;                              // [n_lin][conv_dim][4]
  float *final_norm = nullptr;                          // [H]
  float *mtp_norms = nullptr;                           // [3][H]: pre_fc_norm_embedding, pre_fc_norm_hidden, mtp.norm
  float *rope_cos = nullptr, *rope_sin = nullptr;       // [max_ctx][rotary_dim]
  int rope_ctx = 0;
  void *expert_tables = nullptr;                        // [layers(+mtp)][experts+1] ExpertW
  std::vector<int> slot;                                // per layer: index within its type

  DeviceTensor tensor(const std::string &name) const;
  bool has(const std::string &name) const { return dir.find(name) != nullptr; }
};

// Opens "synth:<preset>[:seed=N]" (filled on the device) or a .binfer path.
// Returns 0, or the reference's exit codes: 1 device/API error or missing
// tensor, 2 bad container / usage.
int model_open(ainfer_device_t dev, const char *spec, int validate_level, DeviceModel **out,
               std::string &err);
void model_close(DeviceModel *m);
// (Re)builds the RoPE tables for at least max_ctx positions.
int model_ensure_rope(DeviceModel *m, int max_ctx, std::string &err);

std::string layer_prefix(int L);

}  // namespace ainfer
