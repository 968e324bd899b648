/* ainfer_cuda.h — device boundary of the B200 decode path (C ABI).
 *
 * This is the layer the decode runtime binds in place of the Level Zero calls
 * the reference makes from its token loop. Each entry point names the
 * reference call it replaces (paths relative to the reference project root).
 * Plain pointers and sizes only; every call returns an int status (0 = ok)
 * and never throws; handles are opaque and owned by the library until the
 * matching destroy/close. One host thread per device handle.
 *
 * Recording model (as tools/decode/decode_l0.cpp:455-493,714-721): kernels
 * are looked up by name, arguments are set by index in member order, a launch
 * appended to a list snapshots the current arguments and is ordered after
 * everything appended before it; a closed list is immutable and replays with
 * no host work. Per-token mutation is only the 16-byte control block in
 * device memory.
 */
#ifndef AINFER_CUDA_H
#define AINFER_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ainfer_device_s *ainfer_device_t;
typedef struct ainfer_kernel_s *ainfer_kernel_t;
typedef struct ainfer_list_s *ainfer_list_t;
typedef struct ainfer_event_s *ainfer_event_t;

enum {
  AINFER_OK = 0,
  AINFER_ERR_INVALID = 1,      /* bad handle, index, size or state            */
  AINFER_ERR_NOT_FOUND = 2,    /* unknown kernel name                          */
  AINFER_ERR_DEVICE = 3,       /* CUDA call failed; see ainfer_last_error      */
  AINFER_ERR_NO_DEVICE = 4,    /* no usable GPU: there is no CPU fallback      */
  AINFER_ERR_TIMEOUT = 5,      /* ainfer_sync ran out of time                  */
  AINFER_ERR_UNSET_ARG = 6,    /* launch appended with an argument never set   */
  AINFER_ERR_OOM = 7
};

/* The per-token control block, tools/decode/decode_l0.cpp:41-43. */
typedef struct ainfer_control {
  int32_t token_id, position, active_length, selected_token;
} ainfer_control;

typedef struct ainfer_device_info {
  char name[64];
  int32_t sm_count, cc_major, cc_minor, l2_bytes_mb;
  uint64_t total_mem, free_mem;
} ainfer_device_info;

/* zeInit/zeDriverGet/zeDeviceGet/zeContextCreate + queue/fence creation,
 * decode_l0.cpp:191-217,455-463. Fails with AINFER_ERR_NO_DEVICE when no GPU
 * is present. */
int ainfer_device_open(int ordinal, ainfer_device_t *out);
int ainfer_device_close(ainfer_device_t dev);
int ainfer_device_get_info(ainfer_device_t dev, ainfer_device_info *info);
/* Text of the last failure on this handle (or of the last failed open when
 * dev is NULL). Valid until the next call on the same thread. */
const char *ainfer_last_error(ainfer_device_t dev);

/* zeMemAllocDevice / zeMemFree, decode_l0.cpp:220-227. align is a power of
 * two, at most 4096. */
int ainfer_mem_alloc(ainfer_device_t dev, size_t bytes, size_t align, void **out);
int ainfer_mem_free(ainfer_device_t dev, void *ptr);
/* Synchronous immediate-list copies and fills (zeCommandListAppendMemoryCopy /
 * MemoryFill on the synchronous immediate list, decode_l0.cpp:239-267,
 * 355-371): ordered after all work already submitted, complete on return. */
int ainfer_memcpy_h2d(ainfer_device_t dev, void *dst, const void *src, size_t bytes);
int ainfer_memcpy_d2h(ainfer_device_t dev, void *dst, const void *src, size_t bytes);
int ainfer_memcpy_d2d(ainfer_device_t dev, void *dst, const void *src, size_t bytes);
int ainfer_mem_fill(ainfer_device_t dev, void *dst, int byte_value, size_t bytes);
/* Pinned host memory for the 4-byte token readback and staged uploads. */
int ainfer_host_alloc(ainfer_device_t dev, size_t bytes, void **out);
int ainfer_host_free(ainfer_device_t dev, void *ptr);
/* Asynchronous copies on the execution queue (ordered with list executes). */
int ainfer_memcpy_h2d_async(ainfer_device_t dev, void *dst, const void *src, size_t bytes);
int ainfer_memcpy_d2h_async(ainfer_device_t dev, void *dst, const void *src, size_t bytes);

/* zeModuleCreate + zeKernelCreate by entry name, decode_l0.cpp:376-447. Every
 * call returns a fresh handle with its own argument storage. */
int ainfer_kernel_get(ainfer_device_t dev, const char *name, ainfer_kernel_t *out);
int ainfer_kernel_release(ainfer_kernel_t k);
/* Enumeration of the kernels the library carries. */
int ainfer_kernel_count(void);
const char *ainfer_kernel_name(int index);
/* Argument count, fixed threads per group and the work items one group covers
 * (rows, heads, ...; 0 = the kernel strides over any group count). */
int ainfer_kernel_query(ainfer_kernel_t k, int *arg_count, int *group_threads, int *items_per_group);
int ainfer_kernel_arg_size(ainfer_kernel_t k, uint32_t index, size_t *size);
/* Largest group count whose groups are all resident at once (occupancy x SM
 * count, with the shared memory the current arguments ask for). Kernels whose
 * groups wait on each other are launched cooperatively and refuse more. No
 * counterpart in the reference: its kernels never synchronise across groups. */
int ainfer_kernel_max_groups(ainfer_kernel_t k, uint32_t *groups);
/* zeKernelSetArgumentValue, decode_l0.cpp:474-480. size must equal the
 * argument's size; value points at the bytes to copy. */
int ainfer_kernel_set_arg(ainfer_kernel_t k, uint32_t index, size_t size, const void *value);

/* zeCommandListCreate / AppendLaunchKernel + AppendBarrier / Close,
 * decode_l0.cpp:464-493,551. */
int ainfer_list_create(ainfer_device_t dev, ainfer_list_t *out);
int ainfer_list_append_launch(ainfer_list_t list, ainfer_kernel_t k, uint32_t group_count);
int ainfer_list_append_memcpy(ainfer_list_t list, void *dst, const void *src, size_t bytes);
int ainfer_list_append_fill(ainfer_list_t list, void *dst, int byte_value, size_t bytes);
int ainfer_list_close(ainfer_list_t list);
int ainfer_list_launch_count(ainfer_list_t list, uint32_t *launches);
int ainfer_list_destroy(ainfer_list_t list);
/* zeCommandQueueExecuteCommandLists, decode_l0.cpp:716: asynchronous. */
int ainfer_list_execute(ainfer_list_t list);
/* Immediate launch outside any list (the SYCL loop's q.submit,
 * tools/decode/decode.cpp:432-477), asynchronous on the execution queue. */
int ainfer_kernel_launch(ainfer_device_t dev, ainfer_kernel_t k, uint32_t group_count);
/* zeFenceHostSynchronize + zeFenceReset, decode_l0.cpp:717-718. timeout_ns ==
 * UINT64_MAX blocks; otherwise polls and returns AINFER_ERR_TIMEOUT. */
int ainfer_sync(ainfer_device_t dev, uint64_t timeout_ns);
/* The 16-byte control copy, decode_l0.cpp:753-756 (synchronous) and an
 * asynchronous form ordered on the execution queue. */
int ainfer_control_write(ainfer_device_t dev, void *dctrl, const ainfer_control *c);
int ainfer_control_write_async(ainfer_device_t dev, void *dctrl, const ainfer_control *c);

/* Device timestamps on the execution queue (the reference times with
 * clock_gettime around blocking executes, decode_l0.cpp:714-721). */
int ainfer_event_create(ainfer_device_t dev, ainfer_event_t *out);
int ainfer_event_record(ainfer_event_t ev);
int ainfer_event_elapsed_ms(ainfer_event_t start, ainfer_event_t stop, float *ms);
int ainfer_event_destroy(ainfer_event_t ev);
/* Number of kernel launches issued on this device handle so far (list
 * replays count every launch they contain). */
int ainfer_launch_counter(ainfer_device_t dev, uint64_t *launches);
/* Writes >126 MB so that the next timed kernel starts with a cold L2. */
int ainfer_flush_l2(ainfer_device_t dev);
/* The raw execution stream (cudaStream_t) for interop with NCCL. */
int ainfer_device_stream(ainfer_device_t dev, void **stream);

/* Router logits + softmax + top-k + renormalised weights + shared-expert gate
 * (the work of the "RouterTopK" kernel) WITHOUT any allocation and without
 * caller-provided scratch. NO COUNTERPART IN THE REFERENCE: its token loop
 * allocates every buffer up front (decode_l0.cpp:270-285) and has no router.
 *
 *   router      [experts][hidden] bf16      shared_gate [hidden] bf16 or NULL
 *   hn          [hidden] fp32 normalised activations
 *   sel_idx     [top_k+1] out: routed expert ids in rank order, then `experts`
 *   sel_w       [top_k+1] out: renormalised weights, then sigmoid(shared gate)
 *   near_gap    [1] out
 * All pointers are device memory. Results are identical to "RouterTopK".
 *
 * The kernel's scratch (logits of all experts and a block counter) lives in a
 * fixed 8192-byte array in device memory that is part of the library image, so
 * the call never calls cudaMalloc/cudaFree or any routine that allocates.
 * Limits and rules:
 *  - experts <= 1024 (what the array holds), top_k <= min(32, experts), hidden
 *    a multiple of 256; anything else returns AINFER_ERR_INVALID with a message.
 *  - The FIRST call on a GPU does one-time set-up (it asks the runtime for the
 *    array's address on that GPU); make that call before starting any stream
 *    capture.
 *  - Every call on one GPU uses the same array. The entry point clears the
 *    counter before each launch; calls that overlap in time on one GPU (other
 *    streams, other handles, other threads) race on the array and must be
 *    serialised by the caller. Calls on this handle's queue are ordered.
 *  - Asynchronous: returns after enqueueing on the handle's queue. */
int ainfer_router_topk_static(ainfer_device_t dev, const void *router, const void *shared_gate,
                              const float *hn, int32_t *sel_idx, float *sel_w, float *near_gap,
                              int32_t experts, int32_t hidden, int32_t top_k);

#ifdef __cplusplus
}
#endif
#endif /* AINFER_CUDA_H */
