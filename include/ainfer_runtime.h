/* ainfer_runtime.h — C ABI of the decode runtime (model-loader, block-executor,
 * token loop, host sampler) that sits on top of ainfer_cuda.h.
 *
 * The reference has no in-process API: its callers drive the decode_l0 binary
 * through argv, stdout lines and a JSON report (tools/http/ainfer_http.py:36,
 * 54-72; tools/e2e/run_e2e.py:30-37). The ainfer_decode executable keeps that
 * process contract; these entry points expose the same loader / executor /
 * token-loop stages in-process so that tests and benchmarks can drive them
 * with plain pointers. Each entry point names the stage of
 * tools/decode/decode_l0.cpp it corresponds to.
 *
 * All calls return 0 on success, otherwise the reference's exit codes:
 * 1 device/API error or missing tensor, 2 usage or bad container, 3 context
 * overflow / internal. ainfer_rt_last_error() gives the message.
 */
#ifndef AINFER_RUNTIME_H
#define AINFER_RUNTIME_H

#include <stddef.h>
#include <stdint.h>

#include "ainfer_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

struct ainfer_sample_params;
typedef struct ainfer_model_s *ainfer_model_t;
typedef struct ainfer_session_s *ainfer_session_t;

const char *ainfer_rt_last_error(void);

/* ---- container (host only, no GPU) ---- */
/* Validation levels: 0 header + directory + span checks (the loader's checks,
 * decode_l0.cpp:127-189), 1 + section CRCs / quant params / overlap, 2 + payload
 * CRCs and trailing SHA-256 (docs/binfer_spec.md section 11). */
int ainfer_binfer_validate(const char *path, int level);
/* Writes a synthetic model of a named shape ("tiny", "mini", "mini-mtp",
 * "small", "full") on the host. Counterpart of tools/binfer.py cmd_quantize
 * (:155-353) with seeded N(0, 0.02) weights in place of a checkpoint. */
int ainfer_synth_write(const char *path, const char *preset, uint64_t seed);
/* Checkpoint ingestion: a SafeTensors file, or a directory holding model.safetensors.index.json
 * and its shards, to a .binfer container. Counterpart of tools/binfer.py cmd_quantize (:155-353)
 * with its policy (:60-64: 2-D tensors to INT4 symmetric g128 with bf16 scales, token embedding
 * and 1-D tensors bf16, vision tower left out) plus this runtime's two bf16 exceptions (router,
 * shared-expert gate). arch_json: the architecture section (the keys ainfer_preset_config_json
 * shows); the directory is checked against it before anything is written. Returns 0 or 2. */
int ainfer_binfer_from_safetensors(const char *src, const char *arch_json, const char *out_path);
/* Architecture JSON of a preset (pointer valid until the next call). */
const char *ainfer_preset_config_json(const char *preset);

/* ---- model-loader (decode_l0.cpp:127-374) ---- */
/* spec: path of a .binfer file, or "synth:<preset>[:seed=N]" to fill the same
 * tensors directly in device memory. */
int ainfer_model_open(ainfer_device_t dev, const char *spec, int validate_level, ainfer_model_t *out);
int ainfer_model_close(ainfer_model_t m);
const char *ainfer_model_config_json(ainfer_model_t m);
int ainfer_model_tensor_count(ainfer_model_t m);
typedef struct ainfer_tensor_info {
  char name[64];
  int32_t storage, ndim;
  uint64_t shape[8];
  void *data;        /* device address */
  uint64_t data_bytes;
  void *scales;      /* device address or NULL */
  uint64_t scale_bytes;
} ainfer_tensor_info;
int ainfer_model_tensor_at(ainfer_model_t m, int index, ainfer_tensor_info *info);
int ainfer_model_tensor(ainfer_model_t m, const char *name, ainfer_tensor_info *info);
/* Total payload + scale bytes resident on the device. */
int ainfer_model_bytes(ainfer_model_t m, uint64_t *payload_bytes, uint64_t *scale_bytes);

/* ---- block-executor + token loop (decode_l0.cpp:270-295,544-825) ---- */
enum {
  AINFER_SESSION_DIAG = 1,            /* per-layer residual dump (AINFER_DUMP0), routed experts, near-tie gaps */
  AINFER_SESSION_PER_LAYER_LISTS = 2, /* one list per layer, fenced one by one, as the reference executes */
  AINFER_SESSION_MULTI_KERNEL = 4,    /* one recorded list per token of stand-alone launches chained by
                                         programmatic dependencies: the default (flag kept for callers) */
  AINFER_SESSION_STAGE_CLOCK = 8,     /* persistent step (implies it): device timestamp after every grid
                                         barrier, read back through the "stage_stamps" buffer (u64 ns) */
  AINFER_SESSION_PERSISTENT = 16      /* ONE persistent cooperative launch per token (DecodeStep) */
};
int ainfer_session_create(ainfer_model_t m, int max_ctx, int flags, ainfer_session_t *out);
int ainfer_session_destroy(ainfer_session_t s);
int ainfer_session_reset(ainfer_session_t s);
/* Device buffers of the session, for state upload/download by tests:
 * "conv", "S", "Kc", "Vc", "Ks", "Vs", "logits", "x", "ctrl", "layer_out",
 * "routed", "near_gap", "history", "stage_stamps". */
int ainfer_session_buffer(ainfer_session_t s, const char *which, void **dptr, uint64_t *bytes);
/* One token at a position; returns the greedy token (4-byte readback). */
int ainfer_session_step(ainfer_session_t s, int token, int pos, int *out_token);
/* P prompt ids from start_pos, then G greedy tokens; device-advanced control
 * block, one readback at the end. gen_ms (optional): device time of the G steps. */
int ainfer_session_generate(ainfer_session_t s, const int *prompt, int P, int G, int start_pos,
                            int *out_tokens, float *gen_ms);
/* Chunked prefill: advances the session's state (DeltaNet state, conv history, INT8 KV cache) over
 * n tokens at positions start_pos.. in passes of up to 192 rows, without logits (chunk orchestration
 * of tools/cmdlist/chunklayer_replay.cpp:366-443). The state afterwards is bit-identical to n calls
 * of ainfer_session_step; follow with ainfer_session_generate(s, &last_prompt_id, 1, G, start_pos + n, ...). */
int ainfer_session_prefill(ainfer_session_t s, const int *tokens, int n, int start_pos);
/* Rows per pass of the next prefill object (1 <= rows, rows x world x top-k <= 2048; default: the
 * largest multiple of 8 within that bound, at most 192). Drops the current prefill object. */
int ainfer_session_prefill_rows(ainfer_session_t s, int rows);
/* Expert parallelism for this session's prefill (config "prefill ... at 8 GPUs with expert
 * parallelism"): every rank prefills its OWN sequence, the MoE block of each pass exchanges rows
 * with the ranks that hold the routed experts (512 / world experts per rank, the all-to-all of
 * ainfer_ep_*), everything else stays on the rank. id128: ainfer_ep_unique_id of one rank, handed
 * to all. Passes hold up to 2048 / (top-k x world) rows of every rank, and the exchanges are collective: every rank must prefill
 * the same number of tokens in the same calls. Call before the first ainfer_session_prefill (a
 * later call drops the prefill object); world == 1 switches back. The state a rank ends with is
 * bit-identical to the one-GPU prefill of the same tokens. */
int ainfer_session_prefill_ep(ainfer_session_t s, const void *id128, int rank, int world);
/* ---- MTP head (multi-token prediction; dataflow of tools/t72/mtp_accept.py:11-16,142-151) ----
 * x = fc . quant([rms1w(embed(next_token)) ; rms1w(h)]) -> one full-attention decoder layer with
 * its own KV cache and MoE -> mtp.norm -> shared lm_head -> argmax. h is the trunk's final
 * residual of the last ainfer_session_step (from_trunk != 0) or the MTP layer's own previous
 * output (chained drafts). The reference only measures acceptance offline and has no
 * draft/verify loop; the loop here is this library's. All three return 2 when the model has
 * no MTP head. */
int ainfer_session_mtp_draft(ainfer_session_t s, int next_token, int pos, int from_trunk, int *draft_token);
int ainfer_session_mtp_logits(ainfer_session_t s, float *host_out);
/* Greedy generation of G tokens with draft_k (1..8) chained drafts per round, each verified by a
 * trunk step (accept iff draft == trunk argmax; a round ends at the first miss). out_tokens are
 * exactly ainfer_session_generate's. stats[3] = {rounds, drafted, accepted}. */
int ainfer_session_generate_mtp(ainfer_session_t s, const int *prompt, int P, int G, int start_pos, int draft_k,
                                int *out_tokens, int *stats);
/* Samples from the last step's logits ON THE DEVICE (kernel SampleToken: the semantics of
 * tools/sample/sampler.h:60-158, see ainfer_sample_token below) and reads back the token and the
 * advanced RNG state (12 bytes instead of 4 V). seen / nseen: ids for the repetition penalty
 * (host array, may be NULL). *rng is the caller's xorshift64* state, as for ainfer_sample_token. */
int ainfer_session_sample(ainfer_session_t s, const struct ainfer_sample_params *p, const int *seen, int nseen,
                          uint64_t *rng, int *out_token);
/* Copies the last step's logits to the host (V floats). */
int ainfer_session_logits(ainfer_session_t s, float *host_out);
int ainfer_session_launches_per_token(ainfer_session_t s, uint64_t *launches);

/* ---- expert-parallel MoE block for a decode batch ----
 * The reference decodes one token on one device (its MLP, tools/decode/decode_l0.cpp:666-674,
 * is dense); this is the sharded form of this library's MoE block: experts split evenly over
 * `world` ranks (one process per GPU), rank r owns batch rows [r*batch/world, (r+1)*batch/world),
 * NCCL send/recv all-to-all for dispatch and return, every token's row bit-identical to the
 * single-GPU decode kernels'. Return codes as above (1 device/NCCL error, 2 usage). */
typedef struct ainfer_ep_s *ainfer_ep_t;
enum { AINFER_EP_ROUTER_BIAS = 1 /* add the "router_bias" buffer to the routed logits (load generators) */ };
/* 128 bytes of a fresh NCCL id: one rank calls it, the caller distributes the bytes. */
int ainfer_ep_unique_id(void *out128);
/* id128 may be NULL when world == 1 (no NCCL is loaded then). batch % world == 0, batch x top-k <= 2048
 * (an expert that receives more than 64 rows is computed as several 64-row problems). */
int ainfer_ep_create(ainfer_model_t m, const void *id128, int rank, int world, int batch, int flags, ainfer_ep_t *out);
int ainfer_ep_destroy(ainfer_ep_t ep);
/* Device buffers: "res" [n][H] f32 input rows of this rank, "x" [n][H] f32 output, "sel_idx"
 * [n][k+1] i32, "sel_w" [n][k+1] f32, "near_gap" [n] f32, "router_bias" [E] f32, "counts" [8] i32
 * of the last layer run (items received; gate/up and down problems of experts with at most 8 rows;
 * gate/up and down problems of experts with more). */
int ainfer_ep_buffer(ainfer_ep_t ep, const char *which, void **dptr, uint64_t *bytes);
/* x = res + MoE(post_attention_norm_L(res)) for the owned rows, then res <- x (so that layers
 * chain); asynchronous on the device's queue. */
int ainfer_ep_moe_layer(ainfer_ep_t ep, int layer);
/* `count` layers from `first`, each feeding the next (res <- x). seg_ms: NULL, or 5 floats that
 * receive the summed device time of route+pack, dispatch exchange, experts, return exchange,
 * shared expert+combine (the call then synchronises after every layer: not for timing the whole). */
int ainfer_ep_moe_stack(ainfer_ep_t ep, int first, int count, float *seg_ms);

/* ---- batched decode ----
 * `batch` sequences advance one token each per step; rank r of `world` owns sequences
 * [r*batch/world, (r+1)*batch/world) with their state and INT8 KV caches (max_ctx tokens each);
 * the MoE layers exchange tokens with the ranks that hold the routed experts (ainfer_ep_*), the
 * rest runs on the owner. Per sequence the arithmetic is the single-sequence token loop's
 * (tools/decode/decode_l0.cpp:742-825), so it decodes to the same tokens in a batch as alone. */
typedef struct ainfer_batch_s *ainfer_batch_t;
int ainfer_batch_create(ainfer_model_t m, const void *id128, int rank, int world, int batch, int max_ctx, int flags,
                        ainfer_batch_t *out);
int ainfer_batch_destroy(ainfer_batch_t b);
/* Device buffers of this rank's n = batch/world sequences: "ctrl" [n][4] i32 {token, position,
 * length, selected}, "out_tok" [n] i32, "logits" [n][V] f32, "x" [n][H] f32 (final residual),
 * state "S", "conv", "Kc", "Vc", "Ks", "Vs" (sequence-major), "router_bias" [E] f32. */
int ainfer_batch_buffer(ainfer_batch_t b, const char *which, void **dptr, uint64_t *bytes);
/* One token for every owned sequence (asynchronous): reads each control block, writes the greedy
 * token to "out_tok" and advances the block, so consecutive calls are a greedy loop. */
int ainfer_batch_step(ainfer_batch_t b);

/* ---- sampler (tools/sample/sampler.h:16-62) ---- */
typedef struct ainfer_sample_params {
  float temp;
  int32_t top_k;
  float top_p;
  float rep_penalty;
  uint64_t seed;
} ainfer_sample_params;
/* In-place repetition penalty over V logits. */
int ainfer_apply_rep_penalty(float *logits, int V, const int *seen, int nseen, float penalty);
/* Returns the selected id; rng is the caller's xorshift64* state; probs_out
 * (optional, V floats) receives the final distribution. */
int ainfer_sample_token(const float *logits, int V, const ainfer_sample_params *p, uint64_t *rng,
                        float *probs_out);

#ifdef __cplusplus
}
#endif
#endif /* AINFER_RUNTIME_H */
