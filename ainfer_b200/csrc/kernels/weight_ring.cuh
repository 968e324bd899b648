// Weight ring: a block streams its contiguous rows of packed INT4 weights (and
// their bf16 scales) from HBM into shared memory with bulk asynchronous copies
// (cp.async.bulk, the untiled TMA path) that complete on mbarriers. One thread
// issues the copies; all 256 threads consume every tile. The copies do not depend on
// activations, so they keep running while the block waits for whatever produces
// its activations (a grid barrier, a staging step): HBM traffic is decoupled
// from the dependency chain of a decode step.
//
// A tile is 16 KB of weights = 256 lanes x 64 bytes = 32768/K whole rows, plus
// the 512 bytes of scales of those rows. (Measured on B200: a block gets about
// one bulk copy per 0.6 us whatever its size up to 32 KB, so 8 KB copies cap a
// 2-blocks-per-SM kernel near 3.7 TB/s while 16 KB copies reach 6.9 TB/s.) Stage i of the ring holds the tile
// with running index t where t % nst == i. full[i] completes when the tile's
// bytes have landed (transaction count); empty[i] completes when all 8 warps
// have copied their bytes into registers (one arrival per warp: arrivals on
// one barrier serialise). Both are waited on with a
// bounded number of polls: a wait that runs out sets the fault word and carries
// on (reading whatever the stage holds), so control flow stays uniform and the
// kernel always terminates; the host reports the fault at the next sync.
#pragma once
#include "common.cuh"
#include "registry.h"

namespace ainfer {

constexpr int kTileBytes = 16384;
constexpr int kTileScaleBytes = 512;
constexpr int kStageStride = kTileBytes + kTileScaleBytes;
constexpr int kMaxStages = 12;
constexpr uint32_t kRingSpinLimit = 1u << 18;

// Contiguous rows of one matrix, dotted with one staged activation vector.
struct RowSeg {
  const uint8_t *P;   // packed nibbles of the segment's first row
  const uint16_t *S;  // bf16 scales of the segment's first row
  int32_t nrows;
  int32_t vec;        // staged activation vector this segment is dotted with
  int32_t trow;       // first row of this segment in the t[][] scratch
  int32_t row0;       // first flat row of this segment in the list (filled by seglist_finalize)
};
constexpr int kMaxSegs = 16;

// A list of segments of matrices with the same K. Lives in shared memory.
struct __align__(16) SegList {
  RowSeg seg[kMaxSegs];
  int32_t nseg;
  int32_t K;
  int32_t ntiles;  // filled by seglist_finalize
  int32_t total;   // rows of all segments together (filled by seglist_finalize)
};

struct Ring {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned char *data;  // nst * kStageStride bytes, 128-byte aligned shared memory
  uint32_t nst;         // stages in use
  uint32_t c_stage;     // stage of the next tile to consume
  uint32_t c_phase;     // parity of that stage's current use
  uint32_t pre;         // leading tiles of the next list that are already in flight
  uint32_t issued;      // tiles issued so far, over all calls (for the drain before an early exit)
  uint32_t fault;       // sticky: 1 a wait ran out, 2 a source was not 16-byte aligned
  // the issuing thread's cursor (kept here so that the issue code is one out-of-line function)
  const SegList *p_list;  // list the next tile comes from
  const SegList *p_next;  // list to continue with when p_list is exhausted (or null)
  int32_t p_tile;         // next tile of p_list
  int32_t p_seg;          // first segment of p_list that can overlap that tile
  uint32_t p_stage, p_phase;  // where it goes
};

// Per-translation-unit pointer to the host-visible fault word (set once per
// device by the library when the device is opened; null = not reported).
static __device__ unsigned int *g_stream_fault_word;
static int set_stream_fault_word(unsigned int *device_ptr) {
  return cudaMemcpyToSymbol(g_stream_fault_word, &device_ptr, sizeof device_ptr) == cudaSuccess ? 0 : 1;
}
static FaultRegistrar g_stream_fault_registrar(set_stream_fault_word);

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long *b, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(b)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(unsigned long long *b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(b)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned long long *b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(b)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_a(uint32_t addr, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(addr), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void mbar_arrive_a(uint32_t addr) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void ring_fault(Ring *ring, uint32_t code) {
  ring->fault = code;
  if (g_stream_fault_word) *reinterpret_cast<volatile unsigned int *>(g_stream_fault_word) = code;
}
// Bounded wait; false (and the fault word set) when it ran out. (Kept inline: a
// call inside the streaming loop would force its live registers to be spilled.)
__device__ __forceinline__ bool mbar_wait_a(Ring *ring, uint32_t addr, uint32_t parity) {
  if (mbar_try_a(addr, parity)) return true;
  // after a first fault no wait in this block spins again: the launch is lost, end it quickly
  const uint32_t limit = *reinterpret_cast<volatile uint32_t *>(&ring->fault) ? 0u : kRingSpinLimit;
#pragma unroll 1
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_a(addr, parity)) return true;
  ring_fault(ring, 1);
  return false;
}
__device__ __forceinline__ bool mbar_wait(Ring *ring, unsigned long long *b, uint32_t parity) {
  return mbar_wait_a(ring, smem_addr(b), parity);
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, unsigned long long *b) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(b))
               : "memory");
}

// Called by every thread once, before the first use. `data` is nst*kStageStride bytes.
__device__ __forceinline__ void ring_init(Ring *ring, unsigned char *data, int nst) {
  if (threadIdx.x == 0) {
    ring->data = data;
    ring->nst = (uint32_t)nst;
    ring->c_stage = 0;
    ring->c_phase = 0;
    ring->pre = 0;
    ring->issued = 0;
    ring->fault = 0;
    ring->p_list = nullptr;
    ring->p_next = nullptr;
    ring->p_tile = 0;
    ring->p_seg = 0;
    ring->p_stage = 0;
    ring->p_phase = 0;
    for (int i = 0; i < nst; ++i) {
      mbar_init(&ring->full[i], 1);
      mbar_init(&ring->empty[i], blockDim.x / 32);  // one arrival per warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
}

// Flat row numbering and tile count of a list; one thread. A tile is the next
// kTileBytes*2/K rows of the list's segments laid end to end, so it may hold
// pieces of several segments (each piece is one bulk copy).
__device__ __forceinline__ void seglist_finalize(SegList *l) {
  const int rpi = kTileBytes * 2 / l->K;
  int n = 0;
  for (int i = 0; i < l->nseg; ++i) {
    l->seg[i].row0 = n;
    n += l->seg[i].nrows;
  }
  l->total = n;
  l->ntiles = (n + rpi - 1) / rpi;
}

// True when a piece's scales can travel by bulk copy (16-byte aligned source,
// size and offset in the stage); otherwise the consumers read them from global
// memory themselves. Producer and consumers evaluate this on the same values.
__device__ __forceinline__ bool piece_scales_bulk(const uint16_t *src, uint32_t bytes, uint32_t dst_off) {
  return ((reinterpret_cast<uintptr_t>(src) | bytes | dst_off) & 15u) == 0;
}

__device__ __forceinline__ void mbar_expect_tx(unsigned long long *b, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(b)), "r"(bytes)
               : "memory");
}

// The issuing thread's cursor. Between calls it rests in the Ring (shared
// memory); the streaming loop keeps it in registers, because the issue sits on
// the critical path of the warp that also consumes.
struct Producer {
  const SegList *l;   // list the next tile comes from (its successor, if any, is ring->p_next)
  int tile, s;        // next tile of l; first segment of l that can overlap it
  uint32_t stage, phase;

  __device__ __forceinline__ void load(const Ring *ring) {
    l = ring->p_list;
    tile = ring->p_tile;
    s = ring->p_seg;
    stage = ring->p_stage;
    phase = ring->p_phase;
  }
  __device__ __forceinline__ void store(Ring *ring) const {
    ring->p_list = l;
    ring->p_tile = tile;
    ring->p_seg = s;
    ring->p_stage = stage;
    ring->p_phase = phase;
  }
  // Issues the copies of the next tile (moving on to ring->p_next when l is
  // exhausted) into `stage`. Returns false when there is nothing left to issue.
  // Few values live in registers between issues: the list's constants are one
  // 16-byte shared-memory read per issue.
  __device__ __forceinline__ bool issue(Ring *ring, unsigned char *data, uint32_t nst) {
    int4 hdr = l ? *reinterpret_cast<const int4 *>(&l->nseg) : make_int4(0, 128, 0, 0);  // nseg, K, ntiles, total
    if (tile >= hdr.z) {
      const SegList *nx = ring->p_next;
      if (nx == nullptr) return false;
      hdr = *reinterpret_cast<const int4 *>(&nx->nseg);
      if (hdr.z == 0) return false;
      l = nx;
      ring->p_next = nullptr;
      tile = 0;
      s = 0;
    }
    const int nseg = hdr.x, K = hdr.y, total = hdr.w;
    const int rpi = kTileBytes * 2 / K, row_bytes = K / 2, srow = K / 64;
    const int f0 = tile * rpi, f1 = f0 + rpi < total ? f0 + rpi : total;
    unsigned char *dst = data + stage * kStageStride;
    unsigned long long *bar = &ring->full[stage];
    while (s < nseg && l->seg[s].row0 + l->seg[s].nrows <= f0) ++s;
#pragma unroll 1
    for (int i = s; i < nseg; ++i) {
      const RowSeg &sg = l->seg[i];
      if (sg.row0 >= f1) break;
      const int a = sg.row0 > f0 ? sg.row0 : f0;
      const int b = sg.row0 + sg.nrows < f1 ? sg.row0 + sg.nrows : f1;
      const int lr = a - sg.row0, rows = b - a, off = a - f0;
      const uint8_t *src = sg.P + (size_t)lr * row_bytes;
      const uint16_t *ssrc =
          reinterpret_cast<const uint16_t *>(reinterpret_cast<const uint8_t *>(sg.S) + (size_t)lr * srow);
      if (reinterpret_cast<uintptr_t>(src) & 15u) {  // cannot be copied in bulk: report and skip
        ring_fault(ring, 2);
        continue;
      }
      const uint32_t wbytes = (uint32_t)(rows * row_bytes), sbytes = (uint32_t)(rows * srow);
      const bool sb = piece_scales_bulk(ssrc, sbytes, (uint32_t)(off * srow));
      mbar_expect_tx(bar, wbytes + (sb ? sbytes : 0));
      bulk_g2s(dst + (size_t)off * row_bytes, src, wbytes, bar);
      if (sb) bulk_g2s(dst + kTileBytes + (size_t)off * srow, ssrc, sbytes, bar);
    }
    mbar_arrive(bar);
    ++tile;
    if (++stage == nst) {
      stage = 0;
      phase ^= 1u;
    }
    return true;
  }
};

// Stateless form: issues tile `tile` of list l into stage `stage`. Any thread may call it, so
// the streaming kernels deal the tiles to the eight warp leaders in turn: issuing a bulk copy
// costs the issuing thread about 550 cycles (measured on B200; a tile is two copies), far too
// much to leave on one consuming warp's critical path for every tile.
__device__ __forceinline__ void ring_issue_tile(Ring *ring, const SegList *l, int tile, uint32_t stage) {
  const int4 hdr = *reinterpret_cast<const int4 *>(&l->nseg);  // nseg, K, ntiles, total
  const int nseg = hdr.x, K = hdr.y, total = hdr.w;
  const int rpi = kTileBytes * 2 / K, row_bytes = K / 2, srow = K / 64;
  const int f0 = tile * rpi, f1 = f0 + rpi < total ? f0 + rpi : total;
  unsigned char *dst = ring->data + stage * kStageStride;
  unsigned long long *bar = &ring->full[stage];
#pragma unroll 1
  for (int i = 0; i < nseg; ++i) {
    const RowSeg &sg = l->seg[i];
    if (sg.row0 + sg.nrows <= f0) continue;
    if (sg.row0 >= f1) break;
    const int a = sg.row0 > f0 ? sg.row0 : f0;
    const int b = sg.row0 + sg.nrows < f1 ? sg.row0 + sg.nrows : f1;
    const int lr = a - sg.row0, rows = b - a, off = a - f0;
    const uint8_t *src = sg.P + (size_t)lr * row_bytes;
    const uint16_t *ssrc =
        reinterpret_cast<const uint16_t *>(reinterpret_cast<const uint8_t *>(sg.S) + (size_t)lr * srow);
    if (reinterpret_cast<uintptr_t>(src) & 15u) {  // cannot be copied in bulk: report and skip
      ring_fault(ring, 2);
      continue;
    }
    const uint32_t wbytes = (uint32_t)(rows * row_bytes), sbytes = (uint32_t)(rows * srow);
    const bool sb = piece_scales_bulk(ssrc, sbytes, (uint32_t)(off * srow));
    mbar_expect_tx(bar, wbytes + (sb ? sbytes : 0));
    bulk_g2s(dst + (size_t)off * row_bytes, src, wbytes, bar);
    if (sb) bulk_g2s(dst + kTileBytes + (size_t)off * srow, ssrc, sbytes, bar);
  }
  mbar_arrive(bar);
}

// Block-wide form of ring_prefetch for the streaming kernels: every thread calls it (no
// synchronisation inside); the warp leaders issue the leading tiles of `list` in parallel.
// Call when the ring is idle (nothing in flight); ring->pre is set by thread 0.
__device__ __forceinline__ void ring_prefetch_all(Ring *ring, const SegList *list) {
  const uint32_t nst = ring->nst;
  const uint32_t cap = (uint32_t)list->ntiles < nst ? (uint32_t)list->ntiles : nst;
  if ((threadIdx.x & 31) == 0) {
    const uint32_t warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (uint32_t j = warp; j < cap; j += warps) {
      uint32_t st = ring->c_stage + j;
      if (st >= nst) st -= nst;
      ring_issue_tile(ring, list, (int)j, st);
    }
  }
  if (threadIdx.x == 0) {
    ring->pre = cap;
    ring->issued += cap;
  }
}

// Out-of-line form for the places that are not in a streaming loop. One thread.
static __device__ __noinline__ bool ring_issue_next(Ring *ring) {
  Producer pr;
  pr.load(ring);
  const bool ok = pr.issue(ring, ring->data, ring->nst);
  pr.store(ring);
  if (ok) ring->issued += 1;
  return ok;
}

// Points the cursor at the start of `list`, at the consumer's position.
__device__ __forceinline__ void ring_open(Ring *ring, const SegList *list) {
  ring->p_list = list;
  ring->p_tile = 0;
  ring->p_seg = 0;
  ring->p_stage = ring->c_stage;
  ring->p_phase = ring->c_phase;
}

// Tops up the ring with leading tiles of `next` (the list the next block_dot
// call will consume). Call between block_dot calls, when every stage not
// counted in ring->pre is free. One thread; no synchronisation.
__device__ __forceinline__ void ring_prefetch(Ring *ring, const SegList *next) {
  if (ring->pre == 0) ring_open(ring, next);
  ring->p_next = nullptr;
  while (ring->pre < ring->nst && ring->p_list == next && ring->p_tile < next->ntiles) {
    ring_issue_next(ring);
    ring->pre += 1;
  }
}

// Before a block leaves its kernel early or after a fault: waits (bounded) for
// whatever may still be in flight into this block's shared memory, so that the
// block does not retire under a landing copy. One thread.
__device__ __forceinline__ void ring_drain(Ring *ring) {
  const uint32_t end = ring->issued;
  for (uint32_t st = 0; st < ring->nst && st < end; ++st) {
    uint32_t t = end - 1 - ((end - 1 - st) % ring->nst);  // latest issued tile held by stage st
    for (uint32_t i = 0; i < kRingSpinLimit; ++i)
      if (mbar_try(&ring->full[st], (t / ring->nst) & 1u)) break;
  }
}
__device__ __forceinline__ void ring_drain_after_fault(Ring *ring) {
  if (ring->fault != 0) ring_drain(ring);
}

}  // namespace ainfer
