// Implementation of include/ainfer_cuda.h over the CUDA runtime: one stream as
// the execution queue, CUDA graphs as recorded command lists. There is no CPU
// fallback: without a usable GPU ainfer_device_open fails.
#include "../../../include/ainfer_cuda.h"

#include <cuda_runtime.h>
#include <time.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../kernels/registry.h"

#include "../common/router_static.h"

namespace ainfer {
// defined beside the fixed scratch array (k_moe.cu)
cudaError_t router_static_scratch_address(void **ptr);
cudaError_t router_static_launch(cudaStream_t stream, void *scratch, const void *Wr, const void *Wsg,
                                 const float *Hn, int32_t *SelIdx, float *SelW, float *NearGap, int E, int H,
                                 int k);
}  // namespace ainfer

namespace ainfer {

static std::vector<KernelDesc> &registry() {
  static std::vector<KernelDesc> r;
  return r;
}
void register_kernel(const KernelDesc &d) { registry().push_back(d); }
void mark_kernel_early_launch(const char *name) {
  for (auto &d : registry())
    if (std::strcmp(d.name, name) == 0) d.early_launch = 1;
}
static std::vector<FaultHook> &fault_hooks() {
  static std::vector<FaultHook> h;
  return h;
}
void register_fault_hook(FaultHook h) { fault_hooks().push_back(h); }
int fault_hook_count() { return (int)fault_hooks().size(); }
FaultHook fault_hook_at(int i) { return fault_hooks()[(size_t)i]; }
static std::vector<TimelineHook> &timeline_hooks() {
  static std::vector<TimelineHook> h;
  return h;
}
void register_timeline_hook(TimelineHook h) { timeline_hooks().push_back(h); }
int kernel_count() { return (int)registry().size(); }
const KernelDesc *kernel_at(int i) {
  return i >= 0 && i < kernel_count() ? &registry()[i] : nullptr;
}
const KernelDesc *kernel_find(const char *name) {
  for (auto &d : registry())
    if (std::strcmp(d.name, name) == 0) return &d;
  return nullptr;
}

}  // namespace ainfer

using namespace ainfer;

struct ainfer_device_s {
  int ordinal = 0;
  cudaStream_t stream = nullptr;
  std::string err;
  uint64_t launches = 0;
  void *flush_buf = nullptr;
  size_t flush_bytes = 0;
  int sm_count = 0;
  volatile unsigned int *fault_word = nullptr;  // host view of the stream fault word of this GPU
  bool early_launch = true;  // recorded lists use programmatic dependencies (AINFER_NO_EARLY_LAUNCH=1 turns it off)
  std::map<void *, void *> over_aligned;  // blocks handed out above cudaMalloc's 256-byte alignment -> the block to free
  std::mutex alloc_mu;
};

// One host-mapped fault word per GPU for the life of the process: kernels that
// stream weights store a code there when one of their bounded waits runs out.
static volatile unsigned int *g_fault_words[64];
static int fault_word_setup(int ordinal, volatile unsigned int **out) {
  if (ordinal < 0 || ordinal >= 64) return 1;
  if (!g_fault_words[ordinal]) {
    unsigned int *h = nullptr, *d = nullptr;
    if (cudaHostAlloc((void **)&h, 64, cudaHostAllocMapped) != cudaSuccess) return 1;
    *h = 0;
    if (cudaHostGetDevicePointer((void **)&d, h, 0) != cudaSuccess) return 1;
    for (int i = 0; i < fault_hook_count(); ++i)
      if (fault_hook_at(i)(d) != 0) return 1;
    g_fault_words[ordinal] = h;
  }
  *out = g_fault_words[ordinal];
  return 0;
}
#ifdef AINFER_TIMELINE
// Event buffer of the timeline build, one per GPU: 2 header words + kTimelineCap (enter, go) pairs.
constexpr size_t kTimelineCap = 1u << 18;
static unsigned long long *g_timeline_bufs[64];
static int timeline_setup(int ordinal) {
  if (ordinal < 0 || ordinal >= 64) return 1;
  if (g_timeline_bufs[ordinal]) return 0;
  unsigned long long *d = nullptr;
  if (cudaMalloc((void **)&d, (2 + 2 * kTimelineCap) * 8) != cudaSuccess) return 1;
  const unsigned long long hdr[2] = {0, kTimelineCap};
  if (cudaMemcpy(d, hdr, sizeof hdr, cudaMemcpyHostToDevice) != cudaSuccess) return 1;
  for (TimelineHook h : timeline_hooks())
    if (h(d) != 0) return 1;
  g_timeline_bufs[ordinal] = d;
  return 0;
}
// Not part of the product ABI: exported by timeline builds for the profiling script.
extern "C" int ainfer_timeline_read(int ordinal, unsigned long long *out_pairs, size_t cap_pairs, size_t *n_out,
                                    int reset) {
  if (ordinal < 0 || ordinal >= 64 || !g_timeline_bufs[ordinal]) return 1;
  cudaSetDevice(ordinal);
  cudaDeviceSynchronize();
  unsigned long long hdr[2];
  if (cudaMemcpy(hdr, g_timeline_bufs[ordinal], sizeof hdr, cudaMemcpyDeviceToHost) != cudaSuccess) return 1;
  size_t n = (size_t)(hdr[0] < hdr[1] ? hdr[0] : hdr[1]);
  if (n > cap_pairs) n = cap_pairs;
  if (n && cudaMemcpy(out_pairs, g_timeline_bufs[ordinal] + 2, n * 16, cudaMemcpyDeviceToHost) != cudaSuccess)
    return 1;
  *n_out = n;
  if (reset) {
    const unsigned long long zero = 0;
    cudaMemcpy(g_timeline_bufs[ordinal], &zero, 8, cudaMemcpyHostToDevice);
  }
  return 0;
}
#endif

struct ainfer_kernel_s {
  ainfer_device_t dev;
  const KernelDesc *desc;
  bool carveout_set = false;
  std::vector<unsigned char> args;
  std::vector<bool> set;
};
struct ainfer_list_s {
  ainfer_device_t dev;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  cudaGraphNode_t last = nullptr;
  bool has_last = false;
  bool last_is_kernel = false;
  bool closed = false;
  uint32_t launches = 0;
};
struct ainfer_event_s {
  ainfer_device_t dev;
  cudaEvent_t ev;
};

static thread_local std::string g_open_err;

static int fail(ainfer_device_t dev, int code, const std::string &msg) {
  if (dev) dev->err = msg;
  else g_open_err = msg;
  return code;
}
#define CU(dev, expr)                                                                         \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess) {                                                                  \
      char _b[512];                                                                           \
      std::snprintf(_b, sizeof _b, "CUDA error %d (%s) at %s:%d (%s)", (int)_e,               \
                    cudaGetErrorString(_e), __FILE__, __LINE__, #expr);                       \
      return fail(dev, _e == cudaErrorMemoryAllocation ? AINFER_ERR_OOM : AINFER_ERR_DEVICE,  \
                  _b);                                                                        \
    }                                                                                         \
  } while (0)

extern "C" {

int ainfer_device_open(int ordinal, ainfer_device_t *out) {
  if (!out) return fail(nullptr, AINFER_ERR_INVALID, "null out pointer");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    cudaGetLastError();
    return fail(nullptr, AINFER_ERR_NO_DEVICE,
                std::string("no CUDA device available (") +
                    (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0") +
                    "); this library has no CPU fallback");
  }
  if (ordinal < 0 || ordinal >= n) return fail(nullptr, AINFER_ERR_INVALID, "bad device ordinal");
  ainfer_device_t d = new ainfer_device_s;
  d->ordinal = ordinal;
  CU(nullptr, cudaSetDevice(ordinal));
  cudaDeviceProp pr;
  CU(nullptr, cudaGetDeviceProperties(&pr, ordinal));
  d->sm_count = pr.multiProcessorCount;
  if (pr.major < 10) {
    delete d;
    return fail(nullptr, AINFER_ERR_NO_DEVICE,
                "device is not sm_100 class: kernels are built for sm_100a only");
  }
  CU(nullptr, cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
  {
    const char *off = std::getenv("AINFER_NO_EARLY_LAUNCH");
    d->early_launch = !(off && off[0] == '1');
  }
  if (fault_word_setup(ordinal, &d->fault_word) != 0) {
    cudaGetLastError();
    cudaStreamDestroy(d->stream);
    delete d;
    return fail(nullptr, AINFER_ERR_DEVICE, "could not set up the stream fault word");
  }
#ifdef AINFER_TIMELINE
  if (timeline_setup(ordinal) != 0) {
    cudaGetLastError();
    cudaStreamDestroy(d->stream);
    delete d;
    return fail(nullptr, AINFER_ERR_DEVICE, "could not set up the timeline buffer");
  }
#endif
  *out = d;
  return AINFER_OK;
}

int ainfer_device_close(ainfer_device_t dev) {
  if (!dev) return AINFER_ERR_INVALID;
  cudaSetDevice(dev->ordinal);
  cudaStreamSynchronize(dev->stream);
  if (dev->flush_buf) cudaFree(dev->flush_buf);
  cudaStreamDestroy(dev->stream);
  delete dev;
  return AINFER_OK;
}

int ainfer_device_get_info(ainfer_device_t dev, ainfer_device_info *info) {
  if (!dev || !info) return AINFER_ERR_INVALID;
  cudaDeviceProp pr;
  CU(dev, cudaGetDeviceProperties(&pr, dev->ordinal));
  std::memset(info, 0, sizeof *info);
  std::snprintf(info->name, sizeof info->name, "%s", pr.name);
  info->sm_count = pr.multiProcessorCount;
  info->cc_major = pr.major;
  info->cc_minor = pr.minor;
  info->l2_bytes_mb = pr.l2CacheSize >> 20;
  size_t fr = 0, tot = 0;
  CU(dev, cudaSetDevice(dev->ordinal));
  CU(dev, cudaMemGetInfo(&fr, &tot));
  info->total_mem = tot;
  info->free_mem = fr;
  return AINFER_OK;
}

const char *ainfer_last_error(ainfer_device_t dev) {
  return dev ? dev->err.c_str() : g_open_err.c_str();
}

int ainfer_mem_alloc(ainfer_device_t dev, size_t bytes, size_t align, void **out) {
  if (!dev || !out) return AINFER_ERR_INVALID;
  if (align > 4096 || (align & (align - 1))) return fail(dev, AINFER_ERR_INVALID, "bad alignment");
  CU(dev, cudaSetDevice(dev->ordinal));
  if (align <= 256) {
    CU(dev, cudaMalloc(out, bytes ? bytes : 1));  // cudaMalloc returns >= 256-byte aligned blocks
    return AINFER_OK;
  }
  // a larger alignment: allocate with slack and hand out the aligned address inside the block
  void *raw = nullptr;
  CU(dev, cudaMalloc(&raw, (bytes ? bytes : 1) + align));
  void *al = (void *)(((uintptr_t)raw + align - 1) & ~(uintptr_t)(align - 1));
  if (al != raw) {
    std::lock_guard<std::mutex> g(dev->alloc_mu);
    dev->over_aligned[al] = raw;
  }
  *out = al;
  return AINFER_OK;
}
int ainfer_mem_free(ainfer_device_t dev, void *ptr) {
  if (!dev) return AINFER_ERR_INVALID;
  CU(dev, cudaSetDevice(dev->ordinal));
  {
    std::lock_guard<std::mutex> g(dev->alloc_mu);
    auto it = dev->over_aligned.find(ptr);
    if (it != dev->over_aligned.end()) {
      ptr = it->second;
      dev->over_aligned.erase(it);
    }
  }
  CU(dev, cudaFree(ptr));
  return AINFER_OK;
}
int ainfer_memcpy_h2d(ainfer_device_t dev, void *dst, const void *src, size_t bytes) {
  if (!dev) return AINFER_ERR_INVALID;
  CU(dev, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, dev->stream));
  CU(dev, cudaStreamSynchronize(dev->stream));
  return AINFER_OK;
}
int ainfer_memcpy_d2h(ainfer_device_t dev, void *dst, const void *src, size_t bytes) {
  if (!dev) return AINFER_ERR_INVALID;
  CU(dev, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, dev->stream));
  CU(dev, cudaStreamSynchronize(dev->stream));
  return AINFER_OK;
}
int ainfer_memcpy_d2d(ainfer_device_t dev, void *dst, const void *src, size_t bytes) {
  if (!dev) return AINFER_ERR_INVALID;
  CU(dev, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, dev->stream));
  CU(dev, cudaStreamSynchronize(dev->stream));
  return AINFER_OK;
}
int ainfer_mem_fill(ainfer_device_t dev, void *dst, int byte_value, size_t bytes) {
  if (!dev) return AINFER_ERR_INVALID;
  CU(dev, cudaMemsetAsync(dst, byte_value, bytes, dev->stream));
  CU(dev, cudaStreamSynchronize(dev->stream));
  return AINFER_OK;
}
int ainfer_host_alloc(ainfer_device_t dev, size_t bytes, void **out) {
  if (!dev || !out) return AINFER_ERR_INVALID;
  CU(dev, cudaMallocHost(out, bytes ? bytes : 1));
  return AINFER_OK;
}
int ainfer_host_free(ainfer_device_t dev, void *ptr) {
  if (!dev) return AINFER_ERR_INVALID;
  CU(dev, cudaFreeHost(ptr));
  return AINFER_OK;
}
int ainfer_memcpy_h2d_async(ainfer_device_t dev, void *dst, const void *src, size_t bytes) {
  if (!dev) return AINFER_ERR_INVALID;
  CU(dev, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, dev->stream));
  return AINFER_OK;
}
int ainfer_memcpy_d2h_async(ainfer_device_t dev, void *dst, const void *src, size_t bytes) {
  if (!dev) return AINFER_ERR_INVALID;
  CU(dev, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, dev->stream));
  return AINFER_OK;
}

int ainfer_kernel_count(void) { return kernel_count(); }
const char *ainfer_kernel_name(int index) {
  const KernelDesc *d = kernel_at(index);
  return d ? d->name : nullptr;
}
int ainfer_kernel_get(ainfer_device_t dev, const char *name, ainfer_kernel_t *out) {
  if (!dev || !name || !out) return AINFER_ERR_INVALID;
  const KernelDesc *d = kernel_find(name);
  if (!d) return fail(dev, AINFER_ERR_NOT_FOUND, std::string("entry ") + name + " not found");
  ainfer_kernel_t k = new ainfer_kernel_s;
  k->dev = dev;
  k->desc = d;
  k->args.assign(d->args_size, 0);
  k->set.assign(d->nfields, false);
  *out = k;
  return AINFER_OK;
}
int ainfer_kernel_release(ainfer_kernel_t k) {
  if (!k) return AINFER_ERR_INVALID;
  delete k;
  return AINFER_OK;
}
int ainfer_kernel_query(ainfer_kernel_t k, int *arg_count, int *group_threads, int *items) {
  if (!k) return AINFER_ERR_INVALID;
  if (arg_count) *arg_count = k->desc->nfields;
  if (group_threads) *group_threads = k->desc->threads;
  if (items) *items = k->desc->items_per_group;
  return AINFER_OK;
}
int ainfer_kernel_arg_size(ainfer_kernel_t k, uint32_t index, size_t *size) {
  if (!k || !size || index >= (uint32_t)k->desc->nfields) return AINFER_ERR_INVALID;
  *size = k->desc->fields[index].size;
  return AINFER_OK;
}
int ainfer_kernel_set_arg(ainfer_kernel_t k, uint32_t index, size_t size, const void *value) {
  if (!k) return AINFER_ERR_INVALID;
  if (index >= (uint32_t)k->desc->nfields)
    return fail(k->dev, AINFER_ERR_INVALID, std::string("setArg index out of range for ") + k->desc->name);
  const ArgField &f = k->desc->fields[index];
  if (size != f.size || !value) {
    char b[160];
    std::snprintf(b, sizeof b, "setArg %u of %s: size %zu, expected %u", index, k->desc->name, size,
                  f.size);
    return fail(k->dev, AINFER_ERR_INVALID, b);
  }
  std::memcpy(k->args.data() + f.offset, value, size);
  k->set[index] = true;
  return AINFER_OK;
}

// The dynamic shared-memory limit is a property of the function, not of one launch: only ever
// raise it, so that a recorded launch with a larger request stays valid after a later, smaller
// one was recorded.
static cudaError_t raise_smem_limit(const void *fn, uint32_t smem) {
  static std::mutex mu;
  static std::map<const void *, uint32_t> raised;
  std::lock_guard<std::mutex> lock(mu);
  uint32_t &cur = raised[fn];
  if (smem <= cur) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) cur = smem;
  return e;
}

static int check_launch(ainfer_kernel_t k, uint32_t groups, uint32_t *smem) {
  for (int i = 0; i < k->desc->nfields; ++i)
    if (!k->set[i]) {
      char b[160];
      std::snprintf(b, sizeof b, "launch of %s with argument %d never set", k->desc->name, i);
      return fail(k->dev, AINFER_ERR_UNSET_ARG, b);
    }
  if (groups == 0) return fail(k->dev, AINFER_ERR_INVALID, "group count 0");
  *smem = k->desc->smem_fn ? k->desc->smem_fn(k->args.data()) : k->desc->smem_bytes;
  // Every kernel asks for the same L1/shared-memory split (all shared): consecutive kernels of a
  // decode step then never make an SM wait for the split to be changed.
  if (!k->carveout_set) {
    if (cudaFuncSetAttribute(k->desc->fn, cudaFuncAttributePreferredSharedMemoryCarveout,
                             (int)cudaSharedmemCarveoutMaxShared) != cudaSuccess)
      cudaGetLastError();
    k->carveout_set = true;
  }
  if (*smem > 16 * 1024) {  // static + dynamic may pass 48 KB: opt in early
    cudaError_t e = raise_smem_limit(k->desc->fn, *smem);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(k->dev, AINFER_ERR_INVALID, std::string("shared memory request too large for ") + k->desc->name);
    }
  }
  if (k->desc->cooperative) {
    // blocks of such a kernel wait on each other: every group must be resident at once
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k->desc->fn, k->desc->threads, *smem);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(k->dev, AINFER_ERR_DEVICE, std::string("occupancy query failed for ") + k->desc->name);
    }
    if ((long)groups > (long)per_sm * k->dev->sm_count) {
      char b[200];
      std::snprintf(b, sizeof b, "%s: %u groups cannot be co-resident (at most %d x %d)", k->desc->name,
                    groups, per_sm, k->dev->sm_count);
      return fail(k->dev, AINFER_ERR_INVALID, b);
    }
  }
  return AINFER_OK;
}

int ainfer_kernel_max_groups(ainfer_kernel_t k, uint32_t *groups) {
  if (!k || !groups) return AINFER_ERR_INVALID;
  uint32_t smem = k->desc->smem_fn ? k->desc->smem_fn(k->args.data()) : k->desc->smem_bytes;
  if (smem > 16 * 1024) {
    if (raise_smem_limit(k->desc->fn, smem) != cudaSuccess) {
      cudaGetLastError();
      return fail(k->dev, AINFER_ERR_INVALID, std::string("shared memory request too large for ") + k->desc->name);
    }
  }
  int per_sm = 0;
  CU(k->dev, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k->desc->fn, k->desc->threads, smem));
  *groups = (uint32_t)per_sm * (uint32_t)k->dev->sm_count;
  return AINFER_OK;
}

int ainfer_kernel_launch(ainfer_device_t dev, ainfer_kernel_t k, uint32_t groups) {
  if (!dev || !k) return AINFER_ERR_INVALID;
  uint32_t smem = 0;
  CU(dev, cudaSetDevice(dev->ordinal));  // function attributes and launches go to the current device
  int r = check_launch(k, groups, &smem);
  if (r) return r;
  void *params[1] = {k->args.data()};
  if (k->desc->cooperative)
    CU(dev, cudaLaunchCooperativeKernel(k->desc->fn, dim3(groups), dim3(k->desc->threads), params, smem, dev->stream));
  else
    CU(dev, cudaLaunchKernel(k->desc->fn, dim3(groups), dim3(k->desc->threads), params, smem, dev->stream));
  dev->launches += 1;
  return AINFER_OK;
}

int ainfer_list_create(ainfer_device_t dev, ainfer_list_t *out) {
  if (!dev || !out) return AINFER_ERR_INVALID;
  ainfer_list_t l = new ainfer_list_s;
  l->dev = dev;
  cudaError_t e = cudaGraphCreate(&l->graph, 0);
  if (e != cudaSuccess) {
    delete l;
    return fail(dev, AINFER_ERR_DEVICE, std::string("list create failed: ") + cudaGetErrorString(e));
  }
  *out = l;
  return AINFER_OK;
}
static const cudaGraphNode_t *deps(ainfer_list_t l) { return l->has_last ? &l->last : nullptr; }

int ainfer_list_append_launch(ainfer_list_t l, ainfer_kernel_t k, uint32_t groups) {
  if (!l || !k) return AINFER_ERR_INVALID;
  if (l->closed) return fail(l->dev, AINFER_ERR_INVALID, "append to a closed list");
  uint32_t smem = 0;
  CU(l->dev, cudaSetDevice(l->dev->ordinal));
  int r = check_launch(k, groups, &smem);
  if (r) return r;
  void *params[1] = {k->args.data()};
  cudaKernelNodeParams np;
  std::memset(&np, 0, sizeof np);
  np.func = const_cast<void *>(k->desc->fn);
  np.gridDim = dim3(groups);
  np.blockDim = dim3(k->desc->threads);
  np.sharedMemBytes = smem;
  np.kernelParams = params;
  cudaGraphNode_t node;
  if (k->desc->early_launch && l->has_last && l->last_is_kernel && l->dev->early_launch) {
    // Programmatic dependency: this kernel may start while its predecessor still runs (its
    // blocks wait in griddepcontrol.wait before touching dependent data), which hides launch
    // latency and lets a GEMV start streaming its weights early.
    alignas(cudaGraphNodeParams) unsigned char gp_raw[sizeof(cudaGraphNodeParams)];
    std::memset(gp_raw, 0, sizeof gp_raw);
    cudaGraphNodeParams &gp = *reinterpret_cast<cudaGraphNodeParams *>(gp_raw);
    gp.type = cudaGraphNodeTypeKernel;
    gp.kernel.func = const_cast<void *>(k->desc->fn);
    gp.kernel.gridDim = dim3(groups);
    gp.kernel.blockDim = dim3(k->desc->threads);
    gp.kernel.sharedMemBytes = smem;
    gp.kernel.kernelParams = params;
    cudaGraphEdgeData ed = {};
    ed.from_port = cudaGraphKernelNodePortProgrammatic;
    ed.to_port = cudaGraphKernelNodePortDefault;
    ed.type = cudaGraphDependencyTypeProgrammatic;
    CU(l->dev, cudaGraphAddNode_v2(&node, l->graph, &l->last, &ed, 1, &gp));
  } else {
    CU(l->dev, cudaGraphAddKernelNode(&node, l->graph, deps(l), l->has_last ? 1 : 0, &np));
  }
  if (k->desc->cooperative) {
    cudaKernelNodeAttrValue v;
    std::memset(&v, 0, sizeof v);
    v.cooperative = 1;
    CU(l->dev, cudaGraphKernelNodeSetAttribute(node, cudaKernelNodeAttributeCooperative, &v));
  }
  l->last = node;
  l->has_last = true;
  l->last_is_kernel = true;
  l->launches += 1;
  return AINFER_OK;
}
int ainfer_list_append_memcpy(ainfer_list_t l, void *dst, const void *src, size_t bytes) {
  if (!l) return AINFER_ERR_INVALID;
  if (l->closed) return fail(l->dev, AINFER_ERR_INVALID, "append to a closed list");
  cudaGraphNode_t node;
  CU(l->dev, cudaGraphAddMemcpyNode1D(&node, l->graph, deps(l), l->has_last ? 1 : 0, dst, src, bytes,
                                      cudaMemcpyDeviceToDevice));
  l->last = node;
  l->has_last = true;
  l->last_is_kernel = false;
  return AINFER_OK;
}
int ainfer_list_append_fill(ainfer_list_t l, void *dst, int byte_value, size_t bytes) {
  if (!l) return AINFER_ERR_INVALID;
  if (l->closed) return fail(l->dev, AINFER_ERR_INVALID, "append to a closed list");
  cudaMemsetParams mp;
  std::memset(&mp, 0, sizeof mp);
  mp.dst = dst;
  mp.value = (unsigned)byte_value & 0xFF;
  mp.elementSize = 1;
  mp.width = bytes;
  mp.height = 1;
  mp.pitch = bytes;
  cudaGraphNode_t node;
  CU(l->dev, cudaGraphAddMemsetNode(&node, l->graph, deps(l), l->has_last ? 1 : 0, &mp));
  l->last_is_kernel = false;
  l->last = node;
  l->has_last = true;
  return AINFER_OK;
}
int ainfer_list_close(ainfer_list_t l) {
  if (!l) return AINFER_ERR_INVALID;
  if (l->closed) return fail(l->dev, AINFER_ERR_INVALID, "list already closed");
  CU(l->dev, cudaSetDevice(l->dev->ordinal));
  CU(l->dev, cudaGraphInstantiate(&l->exec, l->graph, 0));
  l->closed = true;
  return AINFER_OK;
}
int ainfer_list_launch_count(ainfer_list_t l, uint32_t *launches) {
  if (!l || !launches) return AINFER_ERR_INVALID;
  *launches = l->launches;
  return AINFER_OK;
}
int ainfer_list_destroy(ainfer_list_t l) {
  if (!l) return AINFER_ERR_INVALID;
  if (l->exec) cudaGraphExecDestroy(l->exec);
  if (l->graph) cudaGraphDestroy(l->graph);
  delete l;
  return AINFER_OK;
}
int ainfer_list_execute(ainfer_list_t l) {
  if (!l) return AINFER_ERR_INVALID;
  if (!l->closed) return fail(l->dev, AINFER_ERR_INVALID, "execute of a list that is not closed");
  CU(l->dev, cudaSetDevice(l->dev->ordinal));
  CU(l->dev, cudaGraphLaunch(l->exec, l->dev->stream));
  l->dev->launches += l->launches;
  return AINFER_OK;
}

// Sticky: once a kernel reported a stream fault, every later sync fails.
static int stream_fault_check(ainfer_device_t dev) {
  unsigned int code = dev->fault_word ? *dev->fault_word : 0;
  if (code == 0) return AINFER_OK;
  return fail(dev, AINFER_ERR_DEVICE,
              code == 2 ? "weight stream fault: a weight row address was not 16-byte aligned"
                        : "weight stream fault: a bounded wait on a shared-memory copy ran out");
}

int ainfer_sync(ainfer_device_t dev, uint64_t timeout_ns) {
  if (!dev) return AINFER_ERR_INVALID;
  if (timeout_ns == UINT64_MAX) {
    CU(dev, cudaStreamSynchronize(dev->stream));
    return stream_fault_check(dev);
  }
  struct timespec t0, t;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  for (;;) {
    cudaError_t e = cudaStreamQuery(dev->stream);
    if (e == cudaSuccess) return stream_fault_check(dev);
    if (e != cudaErrorNotReady) CU(dev, e);
    clock_gettime(CLOCK_MONOTONIC, &t);
    uint64_t el = (uint64_t)(t.tv_sec - t0.tv_sec) * 1000000000ull + (uint64_t)(t.tv_nsec - t0.tv_nsec);
    if (el >= timeout_ns) return fail(dev, AINFER_ERR_TIMEOUT, "sync timed out");
    struct timespec nap = {0, 20000};
    nanosleep(&nap, nullptr);
  }
}

int ainfer_control_write(ainfer_device_t dev, void *dctrl, const ainfer_control *c) {
  return ainfer_memcpy_h2d(dev, dctrl, c, sizeof *c);
}
int ainfer_control_write_async(ainfer_device_t dev, void *dctrl, const ainfer_control *c) {
  return ainfer_memcpy_h2d_async(dev, dctrl, c, sizeof *c);
}

int ainfer_event_create(ainfer_device_t dev, ainfer_event_t *out) {
  if (!dev || !out) return AINFER_ERR_INVALID;
  ainfer_event_t e = new ainfer_event_s;
  e->dev = dev;
  cudaError_t r = cudaEventCreate(&e->ev);
  if (r != cudaSuccess) {
    delete e;
    return fail(dev, AINFER_ERR_DEVICE, cudaGetErrorString(r));
  }
  *out = e;
  return AINFER_OK;
}
int ainfer_event_record(ainfer_event_t ev) {
  if (!ev) return AINFER_ERR_INVALID;
  CU(ev->dev, cudaEventRecord(ev->ev, ev->dev->stream));
  return AINFER_OK;
}
int ainfer_event_elapsed_ms(ainfer_event_t start, ainfer_event_t stop, float *ms) {
  if (!start || !stop || !ms) return AINFER_ERR_INVALID;
  CU(stop->dev, cudaEventSynchronize(stop->ev));
  CU(stop->dev, cudaEventElapsedTime(ms, start->ev, stop->ev));
  return AINFER_OK;
}
int ainfer_event_destroy(ainfer_event_t ev) {
  if (!ev) return AINFER_ERR_INVALID;
  cudaEventDestroy(ev->ev);
  delete ev;
  return AINFER_OK;
}
int ainfer_launch_counter(ainfer_device_t dev, uint64_t *launches) {
  if (!dev || !launches) return AINFER_ERR_INVALID;
  *launches = dev->launches;
  return AINFER_OK;
}
int ainfer_flush_l2(ainfer_device_t dev) {
  if (!dev) return AINFER_ERR_INVALID;
  if (!dev->flush_buf) {
    dev->flush_bytes = (size_t)256 << 20;
    CU(dev, cudaMalloc(&dev->flush_buf, dev->flush_bytes));
  }
  CU(dev, cudaMemsetAsync(dev->flush_buf, 0, dev->flush_bytes, dev->stream));
  return AINFER_OK;
}
int ainfer_device_stream(ainfer_device_t dev, void **stream) {
  if (!dev || !stream) return AINFER_ERR_INVALID;
  *stream = (void *)dev->stream;
  return AINFER_OK;
}

// ---- router + top-k without any allocation (scratch in a fixed device array) ----
// Address of the fixed scratch array on each GPU, looked up once per GPU.
static void *g_router_static_ptr[64];
static std::mutex g_router_static_mu;

int ainfer_router_topk_static(ainfer_device_t dev, const void *router, const void *shared_gate,
                              const float *hn, int32_t *sel_idx, float *sel_w, float *near_gap,
                              int32_t experts, int32_t hidden, int32_t top_k) {
  if (!dev) return AINFER_ERR_INVALID;
  if (!router || !hn || !sel_idx || !sel_w || !near_gap)
    return fail(dev, AINFER_ERR_INVALID, "ainfer_router_topk_static: null pointer argument");
  if (experts < 1 || experts > kRouterStaticMaxExperts)
    return fail(dev, AINFER_ERR_INVALID,
                "ainfer_router_topk_static: experts = " + std::to_string(experts) +
                    " is outside [1, " + std::to_string(kRouterStaticMaxExperts) +
                    "], the size the fixed scratch array was built for");
  if (top_k < 1 || top_k > 32 || top_k > experts)
    return fail(dev, AINFER_ERR_INVALID, "ainfer_router_topk_static: top_k must be in [1, min(32, experts)]");
  if (hidden < 256 || hidden % 256)
    return fail(dev, AINFER_ERR_INVALID, "ainfer_router_topk_static: hidden must be a positive multiple of 256");
  if (dev->ordinal < 0 || dev->ordinal >= 64) return fail(dev, AINFER_ERR_INVALID, "bad device ordinal");
  void *scratch = nullptr;
  CU(dev, cudaSetDevice(dev->ordinal));  // the launch below goes to the current device
  {
    std::lock_guard<std::mutex> lock(g_router_static_mu);
    if (!g_router_static_ptr[dev->ordinal]) {
      // set-up, once per GPU, with that GPU current: where does this GPU keep the array?
      void *p = nullptr;
      cudaError_t e = router_static_scratch_address(&p);
      if (e != cudaSuccess || p == nullptr) {
        cudaGetLastError();
        return fail(dev, AINFER_ERR_DEVICE,
                    std::string("ainfer_router_topk_static: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
      }
      g_router_static_ptr[dev->ordinal] = p;
    }
    scratch = g_router_static_ptr[dev->ordinal];
  }
  cudaError_t e = router_static_launch(dev->stream, scratch, router, shared_gate, hn, sel_idx, sel_w, near_gap,
                                       experts, hidden, top_k);
  if (e != cudaSuccess) return fail(dev, AINFER_ERR_DEVICE, std::string("ainfer_router_topk_static: ") + cudaGetErrorString(e));
  dev->launches += 1;
  return AINFER_OK;
}

}  // extern "C"
