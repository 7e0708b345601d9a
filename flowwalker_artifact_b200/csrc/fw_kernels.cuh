// Device code of the walk engine (sm_100a).
//
// One persistent grid; every warp claims queries from a global atomic counter
// and walks them to completion.  Per step the row of the current vertex is
// swept in 2 KB sub-blocks with aligned 128-bit accesses:
//   * short rows: straight from global memory (four independent loads per lane);
//   * long rows : through a per-warp ring in shared memory filled by TMA bulk
//                 copies (cp.async.bulk + mbarrier), so the next sub-blocks are
//                 in flight while the current one is reduced.
// Stands in for include/walker.cuh:1307-1580, include/sampler.cuh:46-200,
// include/app.cuh:58-152, include/gpu_task.cuh:24-78 and include/myrand.cuh
// of the reference.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flowwalker.h"
#include "fw_spec.cuh"

namespace fwk {

// Bumped with every change of the device code that can move its counters.
#define FW_KERNEL_REVISION "hub-batched-3"

constexpr int kMaxSchema = 64;
constexpr int kWarpsPerCta = 8;
constexpr int kThreads = 32 * kWarpsPerCta;
#ifndef FW_SLOTS
#define FW_SLOTS 16
#endif
#ifndef FW_N2V_SLOTS
#define FW_N2V_SLOTS 1
#endif
// Queries in flight per warp (slot i lives in the registers of lane i), by the kernel's app.
template <int APP>
__host__ __device__ constexpr int slots_of() {
  return APP == FW_APP_NODE2VEC ? FW_N2V_SLOTS : FW_SLOTS;
}
constexpr int kMinClaim = 4;             // queries claimed per atomic, at least
constexpr int kMaxSmemHist = 8192;       // walk-length histogram kept in shared memory up to this d+1
#ifndef FW_STAGES
#define FW_STAGES 2
#endif
#ifndef FW_N2V_MIN_BLOCKS
#define FW_N2V_MIN_BLOCKS 4
#endif
#ifndef FW_MIN_BLOCKS
#define FW_MIN_BLOCKS 3
#endif
constexpr int kStages = FW_STAGES;       // ring depth per warp
constexpr uint32_t kSubBytes = 16u * fw::kQuadsPerSub;  // 2 KB: one ring stage, one bulk copy
// every app sweeps long rows through the shared-memory ring (node2vec's sweep reads plain weights)
template <int APP>
__host__ __device__ constexpr bool uses_ring() { return true; }
constexpr uint32_t kWaitLimit = 1u << 22;  // polls of an mbarrier before giving up

// Build with -DFW_PHASE_TIMERS to make every warp add up the clock cycles it spends in each part
// of its loop (a development aid: where the warps sit, not what the SM is busy with).
#ifdef FW_PHASE_TIMERS
#define FW_PROF(...) __VA_ARGS__
// 0 short-row picks, 1 direct, 2 ring (cycles); 3..5 their counts; 6 sub-blocks of ring rows;
// 7 in-strip picks of long rows (cycles); 8 everything outside the picks (cycles); 9 warp lifetime
static __device__ unsigned long long g_prof[16];
#else
#define FW_PROF(...)
#endif

// Scratch words (uint64) in device memory.
constexpr int kSlotSteps = 0, kSlotScanned = 1, kSlotStatus = 2, kSlotCounter = 3, kSlotHist = 4;

// Hub batching (see hub_kernel): where walkers that arrive at a hub vertex are parked, and what a
// launch that resumes parked walkers works from.  All pointers are device memory.
struct HubArgs {
  const int32_t* hub_ids;   // the hub vertices, ascending; a vertex is a hub iff its row has >= min_degree edges
  int32_t n_hubs;
  int32_t classes;          // walkers of a hub that may share a sweep: 1, or MetaPath's schema length (those at
                            // the same step modulo it want the same label); a batch is keyed hub * classes + class
  uint32_t min_degree;
  int32_t* kstate;          // steps taken so far by every query that is parked or listed
  const int32_t* list;      // walk kernel: queries to resume (nullptr: fresh queries 0 .. n-1)
  const uint32_t* list_n;   // their number
  int32_t* park_hub;        // parked walkers: hub index ...
  int32_t* park_qi;         // ... and query
  uint32_t* park_n;
  uint32_t* hub_cnt;        // parked walkers per hub
  int32_t* next_list;       // hub kernel: walkers that go on from a vertex that is not a hub
  uint32_t* next_n;
  const int32_t* bucket;    // hub kernel: the parked queries grouped by hub
  const int4* items;        // per item: hub index, first entry in bucket, entries | part << 8 | parts << 16, group
  const uint32_t* items_n;
  const uint16_t* hub_parts;  // parts the sweep of each hub's row is split into (1: one warp sweeps all of it)
  unsigned long long* best64; // split rows: smallest (key << 32 | strip id) per bucket entry over the parts done
  uint32_t* part_done;        // split rows: parts done, per group (index of the group's first item)
  unsigned long long* work; // work counter of this launch
  int32_t* fin;             // per query: the tag of the launch its walk ended in (0: still walking), or nullptr;
  int32_t fin_tag;          // deliver_kernel copies the rows of ended walks to the caller's host table by tag
};

struct WalkArgs {
  HubArgs hub;
  const void* xadj;
  const int32_t* adj;
  const float* weight;
  const int32_t* label;
  int64_t V;
  const int32_t* starts;
  int64_t n;
  int32_t* result;
  unsigned long long* scratch;
  uint64_t qid_base;
  uint64_t qid_stride;  // global id of query i = qid_base + i * qid_stride
  int32_t d;
  uint32_t tp_thresh;
  float inv_p, inv_q;
  float n2v_fmax;  // node2vec: max(1, 1/p, 1/q) with a margin of 1e-5 for rounding
  uint32_t k0, k1;
  uint32_t rk[20];  // the Philox round keys of (k0, k1): fw::philox_round_keys
  int32_t hist_in_smem;
  int32_t schema_len;
  int32_t schema[kMaxSchema];
};

// Per-step context.
struct StepCtx {
  const int4* prim;  // weight (or label) quads of the row: quad q is prim[q]
  const int4* sec;   // neighbour-id quads of the row (node2vec)
  uint32_t nq;       // quads in the row
  uint32_t head;     // first valid edge, relative to quad 0
  uint32_t tail;     // one past the last valid edge, relative to quad 0
  int32_t prev;      // previous vertex or -1
  const int32_t* prow;  // row of prev (node2vec): prow[0 .. plen)
  uint32_t plen;
  int32_t want;      // label wanted (MetaPath)
  // node2vec: where in prev's row the next 32-quad block's search starts (blocks of a row
  // are visited in ascending order, rows are sorted)
  mutable uint32_t from;
  uint32_t* flags;  // 32 words of shared memory owned by this warp
};

// ---- PTX wrappers: mbarrier + bulk async copy (TMA, no multicast) ----

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// global -> this CTA's shared memory; both addresses 16-byte aligned, bytes % 16 == 0
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// Bounded wait: false when the copy did not land within kWaitLimit polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kWaitLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// The same bounded wait as one block of PTX: in the usual case (the copy has landed) it costs the
// test and one taken branch, and the compiler sees no control flow to protect.  1 when the
// phase completed, 0 when kWaitLimit polls went by.
__device__ __forceinline__ uint32_t mbar_wait_inline(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .u32 n;\n\t"
      "mov.u32 n, 0;\n\t"
      "FW_WAIT:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra FW_DONE;\n\t"
      "add.u32 n, n, 1;\n\t"
      "setp.lt.u32 p, n, %3;\n\t"
      "@p bra FW_WAIT;\n\t"
      "FW_DONE:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kWaitLimit)
      : "memory");
  return ok;
}
// expect-tx + bulk copy under a predicate instead of a branch (`go` != 0 in one lane at most)
__device__ __forceinline__ void bulk_g2s_if(uint32_t go, uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.u32 p, %4, 0;\n\t"
      "@p mbarrier.arrive.expect_tx.shared::cta.b64 _, [%3], %2;\n\t"
      "@p cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n\t}" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "r"(go)
      : "memory");
}

// ---- bias of one quad ----

__device__ __forceinline__ float pos(float x) { return fmaxf(x, 0.0f); }

// Warp-cooperative lower bound in the sorted range P[L, R): first index whose value is
// >= target (R if none).  Each round the 32 lanes probe 32 evenly spaced pivots and one
// ballot keeps 1/32 of the range, so a row of 10^6 neighbours takes four rounds where the
// reference's per-thread search (include/gpu_graph.cuh:97-112) takes twenty dependent loads
// per candidate.  All lanes must call it with the same arguments.
__device__ __forceinline__ uint32_t warp_lower_bound(const int32_t* __restrict__ P, uint32_t L, uint32_t R,
                                                     int32_t target, uint32_t lane) {
  while (R - L > 32u) {
    const uint32_t step = (R - L + 31u) >> 5;
    uint32_t idx = L + (lane + 1u) * step - 1u;
    if (idx > R - 1u) idx = R - 1u;
    const int cnt = __popc(__ballot_sync(0xFFFFFFFFu, __ldg(P + idx) < target));  // a prefix of ones
    if (cnt == 32) return R;  // the last pivot is P[R-1]
    L += (uint32_t)cnt * step;
    R = min(R, L + step);
  }
  const bool inb = L + lane < R;
  const int32_t v = inb ? __ldg(P + L + lane) : 0x7FFFFFFF;
  return L + __popc(__ballot_sync(0xFFFFFFFFu, inb && v < target));
}

constexpr uint32_t kN2vStreamMax = 1024;  // windows up to this many entries are streamed, larger ones probed

// node2vec membership for one 32-quad block: which of this lane's four neighbour ids x0..x3
// occur in the previous vertex's sorted row P[0, plen).  Ids of edges outside the current row
// must come in as INT_MIN (before its first edge) or INT_MAX (after its last) so that the
// block's 128 ids are ascending.  Returns the 4-bit mask in the low word and, in the high
// word, where the next block's search starts.
//
// Blocks of a row are visited in ascending order and both rows are sorted, so the part of
// prev's row that matters starts where the previous block's part ended (`from`) and ends at
// the first entry above the block's largest id.  That window is streamed 32 entries at a
// time (one coalesced load per round); every entry finds its place among the block's 128
// ids, which stay in registers, by a binary search with shuffles and flags a match in shared
// memory for the lane that holds it: about two instructions per window entry and no
// dependent global loads per candidate, where the reference probes prev's whole row once
// per candidate (include/gpu_graph.cuh:97-118).  Windows much longer than the block (prev
// a far bigger hub than the current vertex) fall back to per-candidate probes inside the
// window, found by the warp-wide search.  Every lane of the warp must call it.
//
// Not inlined on purpose: it is called from every place that forms a bias, and one copy
// keeps the kernel inside the instruction cache (with the body inlined everywhere the warps
// stalled on instruction fetch 25 cycles per issued instruction).
__device__ __noinline__ unsigned long long n2v_linked_impl(const int32_t* __restrict__ P, uint32_t from,
                                                           uint32_t plen, int32_t x0, int32_t x1, int32_t x2,
                                                           int32_t x3, uint32_t lane, uint32_t* flags) {
  const int32_t kHi = 0x7FFFFFFF, kLo = (int32_t)0x80000000;
  const int32_t lmax = x3 != kHi ? x3 : x2 != kHi ? x2 : x1 != kHi ? x1 : x0 != kHi ? x0 : kLo;
  const int32_t xmax = __reduce_max_sync(0xFFFFFFFFu, lmax);
  bool inb = from + lane < plen;
  int32_t pv = inb ? __ldg(P + from + lane) : kHi;
  uint32_t act = __ballot_sync(0xFFFFFFFFu, inb && pv <= xmax);  // a prefix of ones
  if (act == 0u) return (unsigned long long)from << 32;       // nothing of prev's row in this block's range
  uint32_t whi = from + (uint32_t)__popc(act);
  if (act == 0xFFFFFFFFu) whi = warp_lower_bound(P, from + 32u, plen, xmax + 1, lane);
  uint32_t mine = 0;
  if (whi - from > kN2vStreamMax) {  // warp-uniform
    const int32_t xs[4] = {x0, x1, x2, x3};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (xs[k] == kLo || xs[k] == kHi) continue;
      uint32_t lo = from, hi = whi;
      while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        if (__ldg(P + mid) < xs[k]) lo = mid + 1u; else hi = mid;
      }
      if (lo < whi && __ldg(P + lo) == xs[k]) mine |= 1u << k;
    }
    return ((unsigned long long)whi << 32) | mine;
  }
  flags[lane] = 0u;
  __syncwarp();
  for (uint32_t base = from;;) {
    // pos = number of lanes whose first id is <= pv; the lane before that may hold pv
    uint32_t pos = 0;
#pragma unroll
    for (uint32_t step = 16; step > 0; step >>= 1) {
      const int32_t v = __shfl_sync(0xFFFFFFFFu, x0, (int)(pos + step - 1u));
      pos += v <= pv ? step : 0u;
    }
    pos += __shfl_sync(0xFFFFFFFFu, x0, (int)pos) <= pv ? 1u : 0u;
    const int src = (int)(pos ? pos - 1u : 0u);
    const int32_t y0 = __shfl_sync(0xFFFFFFFFu, x0, src), y1 = __shfl_sync(0xFFFFFFFFu, x1, src);
    const int32_t y2 = __shfl_sync(0xFFFFFFFFu, x2, src), y3 = __shfl_sync(0xFFFFFFFFu, x3, src);
    const uint32_t eq = (y0 == pv ? 1u : 0u) | (y1 == pv ? 2u : 0u) | (y2 == pv ? 4u : 0u) | (y3 == pv ? 8u : 0u);
    if (((act >> lane) & 1u) && pos && eq) atomicOr(&flags[src], eq);
    base += 32u;
    if (base >= whi) break;  // warp-uniform
    inb = base + lane < whi;
    pv = inb ? __ldg(P + base + lane) : kHi;
    act = __ballot_sync(0xFFFFFFFFu, inb);
  }
  __syncwarp();
  mine = flags[lane];
  // Parallel edges: equal ids are adjacent, and a match was flagged on the last lane that
  // starts at or below the value, so earlier copies of the run inherit it from their successor.
  const int32_t nx0 = __shfl_down_sync(0xFFFFFFFFu, x0, 1);
  const bool dup = x0 == x1 || x1 == x2 || x2 == x3 || (lane < 31u && x3 == nx0);
  if (__any_sync(0xFFFFFFFFu, dup && x3 != kHi)) {
    for (;;) {
      const uint32_t nf = __shfl_down_sync(0xFFFFFFFFu, mine, 1);
      uint32_t upd = mine;
      if (lane < 31u && x3 == nx0 && (nf & 1u)) upd |= 8u;
      if (x2 == x3 && (upd & 8u)) upd |= 4u;
      if (x1 == x2 && (upd & 4u)) upd |= 2u;
      if (x0 == x1 && (upd & 2u)) upd |= 1u;
      const bool changed = upd != mine;
      mine = upd;
      if (!__any_sync(0xFFFFFFFFu, changed)) break;
    }
  }
  return ((unsigned long long)whi << 32) | mine;
}

__device__ __forceinline__ uint32_t n2v_linked(const WalkArgs& a, const StepCtx& c, int4 nb, uint32_t q,
                                               bool boundary, uint32_t lane) {
  if (boundary) {  // edges outside the row become -inf / +inf so the 128 ids stay ascending
    const int32_t kHi = 0x7FFFFFFF, kLo = (int32_t)0x80000000;
    const uint32_t r = 4u * q;
    nb.x = r + 0u < c.head ? kLo : r + 0u >= c.tail ? kHi : nb.x;
    nb.y = r + 1u < c.head ? kLo : r + 1u >= c.tail ? kHi : nb.y;
    nb.z = r + 2u < c.head ? kLo : r + 2u >= c.tail ? kHi : nb.z;
    nb.w = r + 3u < c.head ? kLo : r + 3u >= c.tail ? kHi : nb.w;
  }
  const unsigned long long o = n2v_linked_impl(c.prow, c.from, c.plen, nb.x, nb.y, nb.z, nb.w, lane, c.flags);
  c.from = (uint32_t)(o >> 32);
  return (uint32_t)o;
}

// Biases of the four edges of quad q from its raw 16 bytes (`nb`: the four
// neighbour ids and `linked`, which of them are adjacent to the previous vertex: node2vec
// only).  Edges outside the row are NOT masked here.
// CLEAN: the weights are known to be >= 0 and not NaN, so the clamp is skipped.
// An app value with this bit set selects the compact form of the block code (one path per
// block, the boundary masks folded into it) for the same bias.  The largest kernels use it --
// node2vec (plain weights: its sweep of upper bounds, its first step) and the variants that
// share rows between warps: they were measured 13 % and 30 % slower with the two-path blocks.
constexpr int kCompact = 16;
constexpr int kAppPlainCompact = FW_APP_DEEPWALK | kCompact;

template <int APP, bool CLEAN>
__device__ __forceinline__ float4 plain_bias(int4 raw, int32_t want) {
  float4 v;
  if ((APP & (kCompact - 1)) == FW_APP_METAPATH) {  // include/app.cuh:142-147
    v.x = raw.x == want ? 1.0f : 0.0f;
    v.y = raw.y == want ? 1.0f : 0.0f;
    v.z = raw.z == want ? 1.0f : 0.0f;
    v.w = raw.w == want ? 1.0f : 0.0f;
  } else {
    v = make_float4(__int_as_float(raw.x), __int_as_float(raw.y), __int_as_float(raw.z), __int_as_float(raw.w));
    if (!CLEAN) { v.x = pos(v.x); v.y = pos(v.y); v.z = pos(v.z); v.w = pos(v.w); }
  }
  return v;
}

template <int APP, bool CLEAN>
__device__ __forceinline__ float4 quad_bias(const WalkArgs& a, const StepCtx& c, int4 raw, int4 nb, uint32_t q,
                                            uint32_t linked = 0u) {
  if (APP != FW_APP_NODE2VEC) return plain_bias<APP, CLEAN>(raw, c.want);
  float4 v = make_float4(__int_as_float(raw.x), __int_as_float(raw.y), __int_as_float(raw.z), __int_as_float(raw.w));
  if (c.prev >= 0) {  // include/app.cuh:109-122
    const int32_t xs[4] = {nb.x, nb.y, nb.z, nb.w};
    float vs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {  // edges outside the row are zeroed by the caller's mask
      if (xs[k] == c.prev) vs[k] = __fmul_rn(vs[k], a.inv_p);
      else if (!((linked >> k) & 1u)) vs[k] = __fmul_rn(vs[k], a.inv_q);
    }
    v = make_float4(vs[0], vs[1], vs[2], vs[3]);
  }
  if (!CLEAN) { v.x = pos(v.x); v.y = pos(v.y); v.z = pos(v.z); v.w = pos(v.w); }
  return v;
}

// Zeroes the edges of quad q that lie outside [head, tail) (relative edge indices).
__device__ __forceinline__ void mask_quad(float4& v, uint32_t q, uint32_t head, uint32_t tail) {
  const uint32_t x = 4u * q - head, span = tail - head;  // unsigned wrap makes "below head" huge
  v.x = x < span ? v.x : 0.0f;
  v.y = x + 1u < span ? v.y : 0.0f;
  v.z = x + 2u < span ? v.z : 0.0f;
  v.w = x + 3u < span ? v.w : 0.0f;
}

__device__ __forceinline__ float sum4(const float4 v) {
  return __fadd_rn(__fadd_rn(v.x, v.y), __fadd_rn(v.z, v.w));
}
__device__ __forceinline__ float sum_strip(const float S[4]) {
  return __fadd_rn(__fadd_rn(S[0], S[1]), __fadd_rn(S[2], S[3]));
}

// Quad q of the row from global memory, masked when `boundary` (warp-uniform: the
// 32-quad block holds the first or the last quad of the row) says it may need it.
template <int APP, bool CLEAN>
__device__ __forceinline__ float4 load_quad(const WalkArgs& a, const StepCtx& c, uint32_t q, bool boundary) {
  const int4 zero = make_int4(0, 0, 0, 0);
  const bool valid = q < c.nq;
  const int4 raw = valid ? __ldg(c.prim + q) : zero;
  const int4 nb = (APP == FW_APP_NODE2VEC && valid) ? __ldg(c.sec + q) : zero;
  uint32_t linked = 0u;
  if (APP == FW_APP_NODE2VEC && c.prev >= 0) linked = n2v_linked(a, c, nb, q, boundary, threadIdx.x & 31u);
  float4 v = quad_bias<APP, CLEAN>(a, c, raw, nb, q, linked);
  if (boundary) mask_quad(v, q, c.head, c.tail);
  return v;
}

// Quad 32 blk + l of the row, blk <= last_blk (warp-uniform; every lane of the warp calls this).
// Only the row's first and last block can hold a quad that is cut by the row bounds or lies
// past the end; the blocks in between run without bounds tests or masks.
template <int APP, bool CLEAN>
__device__ __forceinline__ float4 block_quad(const WalkArgs& a, const StepCtx& c, uint32_t blk, uint32_t last_blk,
                                             uint32_t l) {
  if (APP == FW_APP_NODE2VEC || (APP & kCompact) != 0)
    return load_quad<APP, CLEAN>(a, c, 32u * blk + l, blk == 0u || blk == last_blk);
  const uint32_t q = 32u * blk + l;
  if (blk != 0u && blk < last_blk) return plain_bias<APP, CLEAN>(__ldg(c.prim + q), c.want);
  // The warp-level barrier is there for the compiler: without it the two paths are folded into
  // one load followed by the masks, and every interior block pays for them again.
  __syncwarp();
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (q < c.nq) {
    v = plain_bias<APP, CLEAN>(__ldg(c.prim + q), c.want);
    mask_quad(v, q, c.head, c.tail);
  }
  return v;
}

// Lane `lane`'s four quads of sub-block b (quads 128 b + 32 j + lane, j = 0..3) from global
// memory: their total bias in the fixed order (S0+S1)+(S2+S3).  Blocks of 32 quads past the
// end of the row are skipped as a warp.
template <int APP, bool CLEAN>
__device__ __forceinline__ float sub_global(const WalkArgs& a, const StepCtx& c, uint32_t b, uint32_t lane) {
  const uint32_t last_blk = (c.nq - 1u) >> 5;
  float S[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t blk = 4u * b + j;
    S[j] = 0.0f;
    if (blk <= last_blk) S[j] = sum4(block_quad<APP, CLEAN>(a, c, blk, last_blk, lane));
  }
  return sum_strip(S);
}

// Sub-block 0 of a row of more than 32 quads.  `more` (warp-uniform): the row has further
// sub-blocks, so blocks 1..3 are interior and need no test at all.
template <int APP, bool CLEAN>
__device__ __forceinline__ float sub_first(const WalkArgs& a, const StepCtx& c, bool more, uint32_t lane) {
  if (APP == FW_APP_NODE2VEC || (APP & kCompact) != 0 || !more) return sub_global<APP, CLEAN>(a, c, 0u, lane);
  const uint32_t last_blk = (c.nq - 1u) >> 5;
  float S[4];
  S[0] = sum4(block_quad<APP, CLEAN>(a, c, 0u, last_blk, lane));
#pragma unroll
  for (int j = 1; j < 4; ++j) S[j] = sum4(plain_bias<APP, CLEAN>(__ldg(c.prim + (32u * j + lane)), c.want));
  return sum_strip(S);
}

// Smallest (key, id) over the warp; ids are unique.
__device__ __forceinline__ void warp_argmin(uint32_t& key, uint32_t& id) {
  const uint32_t m = __reduce_min_sync(0xFFFFFFFFu, key);
  id = __reduce_min_sync(0xFFFFFFFFu, key == m ? id : 0xFFFFFFFFu);
  key = m;
}

// A lane's best candidate so far: key bits, strip id, the pick word of its Philox block and
// the strip's total bias.
struct Best {
  uint32_t key, id, pick;
  float W;
};

// Exact test of one strip: key = E(x) / W.
__device__ __forceinline__ void offer(Best& b, uint32_t x, uint32_t pick_word, float W, uint32_t id) {
  if (W > 0.0f) {
    const uint32_t bits = __float_as_uint(__fdiv_rn(fw::exp_key(x), W));
    if (bits < b.key) { b.key = bits; b.id = id; b.pick = pick_word; b.W = W; }
  }
}

// The same test behind a cheap filter, for the long sweep: E >= clz(x) and, when
// clz(x) == 0, E >= 0.72 * m, so a strip whose lower bound already exceeds
// (best key so far) * W cannot win and its exact key (polynomial + division) is never
// formed.  `bound` may be stale or NaN (nothing found yet): the comparison then lets
// the candidate through.
__device__ __forceinline__ void offer_filtered(Best& b, uint32_t x, uint32_t pick_word, float W, uint32_t id,
                                               float bound) {
  const int g = __clz((int)x);
  const float lower = g ? (float)g : __fmul_rn((float)(x << 1), 0.72f * 0x1p-32f);
  if (W > 0.0f && !(lower > __fmul_rn(__fmul_rn(bound, W), 1.000001f))) offer(b, x, pick_word, W, id);
}

// Per-warp ring state.
struct Ring {
  uint32_t data;    // shared address of stage 0 (stages are contiguous)
  uint32_t bar;     // shared address of mbarrier 0 (8 bytes apart)
  uint32_t parity;  // bit st = parity to wait for on stage st
  bool failed;      // a wait ran out
};

template <int APP>
__device__ __forceinline__ constexpr uint32_t stage_bytes() {
  return kSubBytes;
}

// Issues the bulk copies of sub-block b into stage T (lane 0 only calls this).
template <int APP>
__device__ __forceinline__ void ring_fill(const StepCtx& c, const Ring& ring, uint32_t b, uint32_t T) {
  constexpr uint32_t kSB = stage_bytes<APP>();
  const uint32_t bar = ring.bar + 8u * T;
  mbar_expect_tx(bar, kSB);
  bulk_g2s(ring.data + T * kSB, c.prim + (size_t)b * fw::kQuadsPerSub, kSubBytes, bar);
}

// One interior sub-block b from stage T of the ring: wait for its copy, reduce the lane's
// four quads into A, hand the stage back (refill with sub-block b + kStages, while it is
// still interior).  False when the wait ran out.
template <int APP, bool CLEAN>
__device__ __forceinline__ bool ring_sub(const WalkArgs& a, const StepCtx& c, uint32_t b, uint32_t last_b,
                                         uint32_t lane, Ring& ring, const unsigned char* ring_ptr, const uint32_t T,
                                         float& A) {
  constexpr uint32_t kSB = stage_bytes<APP>();
  const uint32_t bar = ring.bar + 8u * T;
  bool ok = mbar_try_wait(bar, (ring.parity >> T) & 1u) != 0;
  if (!ok) ok = mbar_wait(bar, (ring.parity >> T) & 1u);
  ring.parity ^= 1u << T;
  const int4* st = reinterpret_cast<const int4*>(ring_ptr + T * kSB);
  const int4 zero = make_int4(0, 0, 0, 0);
  int4 raw[4], nb[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) raw[j] = st[lane + 32 * j];
#pragma unroll
  for (int j = 0; j < 4; ++j) nb[j] = APP == FW_APP_NODE2VEC ? st[fw::kQuadsPerSub + lane + 32 * j] : zero;
  float S[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t q = b * fw::kQuadsPerSub + lane + 32u * j;
    uint32_t linked = 0u;
    if (APP == FW_APP_NODE2VEC && c.prev >= 0) linked = n2v_linked(a, c, nb[j], q, false, lane);
    S[j] = sum4(quad_bias<APP, CLEAN>(a, c, raw[j], nb[j], q, linked));
  }
  A = sum_strip(S);
  // Every lane's A is formed (its staged values are consumed) before the stage is refilled.
  if (!__all_sync(0xFFFFFFFFu, ok && A >= 0.0f)) return false;
  if (lane == 0 && b + kStages < last_b) ring_fill<APP>(c, ring, b + kStages, T);
  return true;
}

// ---- the sweep of DeepWalk, PPR and MetaPath: two stages of half a supergroup (4 KB) each ----
//
// A warp sweeping a row is one chain of dependent steps per staged copy: wait, load from shared
// memory, add, hand the stage back.  The SM's throughput on long rows is (warps) x (bytes per
// chain) / (latency of the chain), so the stage is made large -- one bulk copy, one wait and one
// refill per 4 KB, the eight 128-bit loads and the thirty adds of a stage independent of one
// another -- and every row of more than 32 quads goes through the ring from its first quad to its
// last: half h of the row (quads 256 h .. 256 h + 255, the last one as far as the row goes)
// sits in stage h mod 2, supergroup s is halves 2s and 2s+1.  Both stages are filled when the
// row starts, so a row of up to 2,048 neighbours is one round trip to memory, whatever its
// length, and is still in shared memory when the pick inside the winning strip needs it.  The
// row's first and last supergroup are reduced with the boundary masks, the ones in between bare.
constexpr uint32_t kHalfBytes = 2u * kSubBytes;      // one stage
constexpr uint32_t kHalfQuads = 2u * fw::kQuadsPerSub;

// Hub batching: a vertex is a hub from a limit of neighbours on.  The walk kernel of a hub-batched
// call only meets rows below the limit and stages each of them whole: a row of fewer than
// 4 Q - 7 neighbours is at most Q quads however it is aligned.  Two limits are compiled, the
// lower one for calls that bring enough walkers per hub to fill its batches:
// 504 (rows of at most 128 quads, 2 KB stages, four CTAs per SM) and 1,016 (256 quads, 4 KB, three).
constexpr uint32_t kHubLimitLow = 504, kHubLimitHigh = 1016;
__host__ __device__ constexpr uint32_t staged_quads(uint32_t limit) { return (limit + 7u + 3u) / 4u; }
static_assert(staged_quads(kHubLimitLow) == 128u && staged_quads(kHubLimitHigh) == 256u, "one or two sub-blocks per lane");

// Ring bytes per warp by the kernel's app: node2vec keeps the ring of two 2 KB stages.
template <int APP>
__host__ __device__ constexpr uint32_t ring_bytes() {
  return APP == FW_APP_NODE2VEC ? (uint32_t)kStages * kSubBytes : 2u * kHalfBytes;
}

// Bytes of half h of a row of nq quads.
__device__ __forceinline__ uint32_t half_bytes(uint32_t nq, uint32_t h) {
  return 16u * min(kHalfQuads, nq - kHalfQuads * h);
}

// Half h of the row into its stage (lane 0 only calls this; h < number of halves).
__device__ __forceinline__ void half_fill(const StepCtx& c, const Ring& ring, uint32_t h) {
  const uint32_t T = h & 1u, bytes = half_bytes(c.nq, h);
  mbar_expect_tx(ring.bar + 8u * T, bytes);
  bulk_g2s(ring.data + T * kHalfBytes, c.prim + (size_t)h * kHalfQuads, bytes, ring.bar + 8u * T);
}

// Half 2s + T of the row from stage T: the lane's two partial sums (one per sub-block), then the
// stage is handed back with half 2s + T + 2 (while that one is below h_end) by lane 0 alone, and
// only once its own sums exist: a shared-memory load delivers all lanes' values together, so the
// warp has read the whole stage by then.  (The sums are >= 0 always; the test is there to make
// the refill depend on the loads.)  EDGE: the supergroup holds the row's first or last quad --
// quads outside the row (stale bytes of the stage included) are masked, and a half that does
// not exist counts as zero, which leaves the strip's total as the shorter sum would give it.
// `lane_ptr` = the warp's stage 0 + 16 * lane.  Returns 0 when the wait ran out.
template <int APP, bool CLEAN, int T, bool EDGE>
__device__ __forceinline__ uint32_t half_take(const StepCtx& c, uint32_t s, uint32_t n_half, uint32_t h_end,
                                              uint32_t lane, const Ring& ring, const int4* lane_ptr, uint32_t& parity,
                                              float& Alo, float& Ahi) {
  const uint32_t h = 2u * s + T;
  if (EDGE && h >= n_half) {  // warp-uniform
    Alo = 0.0f;
    Ahi = 0.0f;
    return 1u;
  }
  const uint32_t bar = ring.bar + 8u * T;
  const uint32_t ok = mbar_wait_inline(bar, (parity >> T) & 1u);
  parity ^= 1u << T;
  const int4* st = lane_ptr + T * kHalfQuads;
  int4 raw[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) raw[j] = st[32 * j];
  float S[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float4 v = plain_bias<APP, CLEAN>(raw[j], c.want);
    if (EDGE) mask_quad(v, kHalfQuads * h + 32u * j + lane, c.head, c.tail);
    S[j] = sum4(v);
  }
  Alo = sum_strip(S);
  Ahi = sum_strip(S + 4);
  const uint32_t go = (lane == 0u && h + 2u < h_end && Alo >= 0.0f && Ahi >= 0.0f) ? ok : 0u;
  bulk_g2s_if(go, ring.data + T * kHalfBytes, c.prim + (size_t)(h + 2u) * kHalfQuads, half_bytes(c.nq, h + 2u), bar);
  return ok;
}

// One whole supergroup s: both stages, the strip's total in the canonical order (A0+A1)+(A2+A3).
// False when a staged copy did not arrive (looked at once per supergroup: until then the sums
// are formed from whatever the stage holds and dropped, and nothing is refilled).
template <int APP, bool CLEAN, bool EDGE>
__device__ __forceinline__ bool super_turn(const StepCtx& c, uint32_t s, uint32_t n_half, uint32_t h_end,
                                           uint32_t lane, Ring& ring, const int4* lane_ptr, float& W) {
  float A0, A1, A2, A3;
  uint32_t ok = half_take<APP, CLEAN, 0, EDGE>(c, s, n_half, h_end, lane, ring, lane_ptr, ring.parity, A0, A1);
  ok &= half_take<APP, CLEAN, 1, EDGE>(c, s, n_half, h_end, lane, ring, lane_ptr, ring.parity, A2, A3);
  W = __fadd_rn(__fadd_rn(A0, A1), __fadd_rn(A2, A3));
  return __all_sync(0xFFFFFFFFu, ok != 0u);
}

// ---- node2vec: sweep with the membership test only where it can matter ----
//
// bias = w * f with f in {1/p, 1, 1/q}, so a strip's total bias W is at most fmax * sum(w) and
// its key E / W at least E / (fmax * sum(w)).  The sweep therefore adds up the plain weights
// only (no neighbour ids, no membership test) and looks closer only at strips whose optimistic
// key could still beat the best true key so far: a handful per row.  A strip that is skipped has
// a true key above the final minimum, so the result is the one the full evaluation gives.  The reference evaluates the membership test for every
// candidate of every row (include/app.cuh:109-122).

// Exact biases of strip (s, L) spread over the warp: lane t holds edges 2*(t&1), 2*(t&1)+1 of the
// strip's quad t>>1, i.e. the strip's 64 edges in canonical order are lane 0 (b0, b1), lane 1
// (b0, b1), ...  Membership by one binary search over prev's row per edge (two per lane, run side
// by side).  Returns the strip's total in the canonical summation order, identical on all lanes.
template <bool CLEAN>
__device__ __forceinline__ float n2v_strip_exact(const WalkArgs& a, const StepCtx& c, uint32_t s, uint32_t L,
                                                 uint32_t lane, float& b0, float& b1) {
  const uint32_t q = s * fw::kQuadsPerSuper + 32u * (lane >> 1) + L;
  const uint32_t k0 = 2u * (lane & 1u);
  b0 = 0.0f;
  b1 = 0.0f;
  int32_t x0 = 0, x1 = 0;
  const uint32_t r0 = 4u * q + k0;
  const bool v0 = q < c.nq && r0 >= c.head && r0 < c.tail;
  const bool v1 = q < c.nq && r0 + 1u >= c.head && r0 + 1u < c.tail;
  if (q < c.nq) {
    // the lane's two edges are the low or the high half of the quad: one 8-byte load each
    const float2 w = __ldg(reinterpret_cast<const float2*>(c.prim + q) + (lane & 1u));
    const int2 x = __ldg(reinterpret_cast<const int2*>(c.sec + q) + (lane & 1u));
    b0 = w.x; b1 = w.y; x0 = x.x; x1 = x.y;
  }
  // lower bounds of x0 and x1 in prev's row, both searches advancing together
  uint32_t lo0 = 0, hi0 = v0 && x0 != c.prev ? c.plen : 0u;
  uint32_t lo1 = 0, hi1 = v1 && x1 != c.prev ? c.plen : 0u;
  while (lo0 < hi0 || lo1 < hi1) {
    const uint32_t m0 = lo0 + ((hi0 - lo0) >> 1), m1 = lo1 + ((hi1 - lo1) >> 1);
    const int32_t p0 = lo0 < hi0 ? __ldg(c.prow + m0) : 0;
    const int32_t p1 = lo1 < hi1 ? __ldg(c.prow + m1) : 0;
    if (lo0 < hi0) { if (p0 < x0) lo0 = m0 + 1u; else hi0 = m0; }
    if (lo1 < hi1) { if (p1 < x1) lo1 = m1 + 1u; else hi1 = m1; }
  }
  const bool linked0 = v0 && x0 != c.prev && lo0 < c.plen && __ldg(c.prow + lo0) == x0;
  const bool linked1 = v1 && x1 != c.prev && lo1 < c.plen && __ldg(c.prow + lo1) == x1;
  b0 = !v0 ? 0.0f : x0 == c.prev ? __fmul_rn(b0, a.inv_p) : linked0 ? b0 : __fmul_rn(b0, a.inv_q);
  b1 = !v1 ? 0.0f : x1 == c.prev ? __fmul_rn(b1, a.inv_p) : linked1 ? b1 : __fmul_rn(b1, a.inv_q);
  if (!CLEAN) { b0 = pos(b0); b1 = pos(b1); }
  // (w0+w1)+(w2+w3) per quad, (S0+S1)+(S2+S3) per sub-block, (A0+A1)+(A2+A3): a butterfly
  float t = __fadd_rn(b0, b1);
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const float o = __shfl_xor_sync(0xFFFFFFFFu, t, d);
    t = (lane & d) ? __fadd_rn(o, t) : __fadd_rn(t, o);  // same operands in the same order on both lanes
  }
  return t;
}

// node2vec, end of a supergroup: every lane holds the plain-weight total of its strip (Wplain) and
// its random word x (pick word pw).  Each lane forms the optimistic key of its strip,
// E / (fmax * Wplain), which is never above the strip's true key; strips are then evaluated
// exactly in the order of their optimistic keys and only while that key does not exceed the best
// true key so far: usually one or two strips in the first supergroup of a row, none in the others.
// `best` is kept identical on all lanes.
template <bool CLEAN>
__device__ __forceinline__ void n2v_test(const WalkArgs& a, const StepCtx& c, uint32_t s, uint32_t lane,
                                         float Wplain, uint32_t x, uint32_t pw, Best& best) {
  uint32_t klo = 0xFFFFFFFFu;  // optimistic key bits; 0xFFFFFFFF = nothing to evaluate in this lane
  if (Wplain > 0.0f) klo = __float_as_uint(__fdiv_rn(fw::exp_key(x), __fmul_rn(Wplain, a.n2v_fmax)));
#pragma unroll 1
  for (;;) {
    const uint32_t kmin = __reduce_min_sync(0xFFFFFFFFu, klo);
    if (kmin == 0xFFFFFFFFu || kmin > best.key) break;  // equal keys still need a look: the lower id wins
    const uint32_t L = (uint32_t)__ffs((int)__ballot_sync(0xFFFFFFFFu, klo == kmin)) - 1u;
    float b0, b1;
    const float W = n2v_strip_exact<CLEAN>(a, c, s, L, lane, b0, b1);
    const uint32_t xL = __shfl_sync(0xFFFFFFFFu, x, (int)L), pL = __shfl_sync(0xFFFFFFFFu, pw, (int)L);
    if (W > 0.0f) {
      const uint32_t bits = __float_as_uint(__fdiv_rn(fw::exp_key(xL), W));
      const uint32_t id = s * 32u + L;
      if (bits < best.key || (bits == best.key && id < best.id)) { best.key = bits; best.id = id; best.pick = pL; best.W = W; }
    }
    if (lane == L) klo = 0xFFFFFFFFu;  // evaluated
  }
}

// node2vec: inverse-CDF pick inside the winning strip B from its exact biases, spread over the
// warp in canonical order (lane 0 (b0, b1), lane 1 (b0, b1), ...): the first edge whose running
// sum exceeds u * W.
template <bool CLEAN>
__device__ __forceinline__ uint32_t n2v_pick(const WalkArgs& a, const StepCtx& c, uint32_t B, uint32_t pick,
                                             uint32_t lane) {
  const uint32_t sB = B >> 5, lB = B & 31u;
  float b0, b1;
  const float W = n2v_strip_exact<CLEAN>(a, c, sB, lB, lane, b0, b1);
  const float thr = __fmul_rn((float)(pick >> 8) * 0x1p-24f, W);
  float acc = 0.0f;
  uint32_t cnt = 0;
#pragma unroll 1
  for (int t = 0; t < 32; ++t) {
    acc = __fadd_rn(acc, __shfl_sync(0xFFFFFFFFu, b0, t)); cnt += acc <= thr ? 1u : 0u;
    acc = __fadd_rn(acc, __shfl_sync(0xFFFFFFFFu, b1, t)); cnt += acc <= thr ? 1u : 0u;
    if (cnt < 2u * (uint32_t)(t + 1)) break;  // found (warp-uniform)
  }
  if (cnt >= 64u) {  // rounding pushed u * W past the sequential total: the strip's last positive edge
    const uint32_t m1 = __ballot_sync(0xFFFFFFFFu, b1 > 0.0f), m0 = __ballot_sync(0xFFFFFFFFu, b0 > 0.0f);
    const int t1 = 31 - __clz((int)m1), t0 = 31 - __clz((int)m0);  // -1 when the mask is empty
    cnt = t1 >= t0 ? 2u * (uint32_t)t1 + 1u : 2u * (uint32_t)t0;
  }
  // position z = 4 j + k of the strip: quad 512 s + 32 j + l, edge k
  return 4u * (sB * fw::kQuadsPerSuper + 32u * (cnt >> 2) + lB) + (cnt & 3u);
}

// The sweep of node2vec reads plain weights (DeepWalk's bias); its own bias enters per strip.
// Kernel variant (template MODE) of the strip sampler whose warps also share very long rows: kept
// apart because the sharing code costs the plain sweep registers (48 against 40, one CTA per SM less)
// and about 20 % of its throughput; the engine selects it for graphs that have rows long enough to
// leave a tail.
constexpr int kModeStripShared = FW_GROUP_STRIP + 1;
template <int APP, int MODE = kModeStripShared>
struct SweepApp {
  static constexpr int value = APP == FW_APP_NODE2VEC ? kAppPlainCompact
                             : MODE == kModeStripShared ? (APP | kCompact) : APP;
};

// A lane's running state while a row is swept: the partial sums of the current supergroup
// and the Philox block that serves it.
struct SuperAcc {
  float p01, a2;   // A0+A1 and A2 of the supergroup in progress
  uint32_t g, m;   // its Philox block (supergroup index / 3) and word (index mod 3)
  fw::Philox4 r;
};

// Adds sub-block b's partial sum A; at the end of a supergroup (or of the row) forms the strip's
// total (A0+A1)+(A2+A3) and tests its key, behind the lower-bound filter when `filtered`.
template <int APP, bool CLEAN>
__device__ __forceinline__ void absorb(const WalkArgs& a, const StepCtx& c, SuperAcc& s, Best& best, float A,
                                       uint32_t b, bool row_end, bool filtered, uint32_t lane, uint32_t c1,
                                       uint32_t qlo, uint32_t qhi) {
  const uint32_t u = b & 3u;
  if (u == 0u) s.p01 = A;
  else if (u == 1u) s.p01 = __fadd_rn(s.p01, A);
  else if (u == 2u) s.a2 = A;
  if (u == 3u || row_end) {
    const float W = u == 3u ? __fadd_rn(s.p01, __fadd_rn(s.a2, A)) : u == 2u ? __fadd_rn(s.p01, s.a2) : s.p01;
    const uint32_t x = s.m == 0u ? s.r.x : s.m == 1u ? s.r.y : s.r.z;
    const uint32_t id = (b >> 2) * 32u + lane;
    if (APP == FW_APP_NODE2VEC && c.prev >= 0) n2v_test<CLEAN>(a, c, b >> 2, lane, W, x, s.r.w, best);
    else if (filtered) offer_filtered(best, x, s.r.w, W, id, __uint_as_float(__reduce_min_sync(0xFFFFFFFFu, best.key)));
    else offer(best, x, s.r.w, W, id);
    if (!row_end) {
      if (++s.m == 3u) { s.m = 0u; s.r = fw::philox4x32_10((++s.g) * 32u + lane, c1, qlo, qhi, a.k0, a.k1); }
    }
  }
}

// The same for a whole supergroup s whose total W is already formed (never the row's last one).
template <int APP, bool CLEAN>
__device__ __forceinline__ void absorb_super(const WalkArgs& a, const StepCtx& c, SuperAcc& s, Best& best, float W,
                                             uint32_t sg, bool last, uint32_t lane, uint32_t c1, uint32_t qlo,
                                             uint32_t qhi) {
  const uint32_t x = s.m == 0u ? s.r.x : s.m == 1u ? s.r.y : s.r.z;
  if (APP == FW_APP_NODE2VEC && c.prev >= 0) n2v_test<CLEAN>(a, c, sg, lane, W, x, s.r.w, best);
  else offer_filtered(best, x, s.r.w, W, sg * 32u + lane, __uint_as_float(__reduce_min_sync(0xFFFFFFFFu, best.key)));
  if (!last && ++s.m == 3u) { s.m = 0u; s.r = fw::philox4x32_10((++s.g) * 32u + lane, c1, qlo, qhi, a.k0, a.k1); }
}

// Inverse-CDF pick inside the winning strip B: the first of its edges in canonical order (quad j,
// edge k) whose running sum exceeds u * W, u from the pick word.  Zero biases leave the running
// sum unchanged, so counting the sums <= u * W gives that edge's position.  The strip's (up to)
// sixteen quads are loaded side by side, one per lane, and the running sum then walks over them
// by shuffles in the canonical order: one memory round trip instead of one per quad.  Plain
// biases only (node2vec picks with n2v_pick).  Returns the edge index relative to quad 0 of the row.
template <int APP, bool CLEAN, bool FROM_RING = false>
__device__ __forceinline__ uint32_t pick_in_row(const WalkArgs& a, const StepCtx& c, uint32_t B, uint32_t pick,
                                                float W, uint32_t lane, const unsigned char* ring_ptr = nullptr) {
  static_assert(APP != FW_APP_NODE2VEC, "node2vec's pick needs the membership test: n2v_pick");
  const uint32_t sB = B >> 5, lB = B & 31u;
  const float thr = __fmul_rn((float)(pick >> 8) * 0x1p-24f, W);
  const uint32_t last_blk = (c.nq - 1u) >> 5;
  const uint32_t blk0 = 16u * sB;
  const uint32_t nblk = min(16u, last_blk - blk0 + 1u);
  const uint32_t q = 32u * (blk0 + lane) + lB;  // lane j holds the strip's quad j
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (lane < nblk && q < c.nq) {
    // FROM_RING: the row is one supergroup at most and still staged (quad q at 16 q of the ring)
    const int4 raw = FROM_RING ? reinterpret_cast<const int4*>(ring_ptr)[q] : __ldg(c.prim + q);
    v = plain_bias<APP, CLEAN>(raw, c.want);
    mask_quad(v, q, c.head, c.tail);
  }
  float acc = 0.0f;
  uint32_t cnt = 0, j = 0;
#pragma unroll 1
  for (; j < nblk; ++j) {
    const float x = __shfl_sync(0xFFFFFFFFu, v.x, (int)j), y = __shfl_sync(0xFFFFFFFFu, v.y, (int)j);
    const float z = __shfl_sync(0xFFFFFFFFu, v.z, (int)j), w = __shfl_sync(0xFFFFFFFFu, v.w, (int)j);
    // biases are >= 0, so the running sums never decrease: when the quad's last sum is still
    // <= thr all four are, and the quad is passed with one comparison
    const float p0 = __fadd_rn(acc, x), p1 = __fadd_rn(p0, y), p2 = __fadd_rn(p1, z);
    acc = __fadd_rn(p2, w);
    if (acc <= thr) { cnt += 4u; continue; }
    cnt += (p0 <= thr ? 1u : 0u) + (p1 <= thr ? 1u : 0u) + (p2 <= thr ? 1u : 0u);
    break;  // found (warp-uniform)
  }
  if (j == nblk) {
    // rounding pushed u * W past the sequential total: take the strip's last positive edge
    const uint32_t m = (v.x > 0.0f ? 1u : 0u) | (v.y > 0.0f ? 2u : 0u) | (v.z > 0.0f ? 4u : 0u) | (v.w > 0.0f ? 8u : 0u);
    const uint32_t have = __ballot_sync(0xFFFFFFFFu, m != 0u);
    const int top = have ? 31 - __clz((int)have) : 0;
    const uint32_t mt = __shfl_sync(0xFFFFFFFFu, m, top);
    cnt = have ? 4u * (uint32_t)top + (uint32_t)(31 - __clz((int)mt)) : 0u;
  }
  return 4u * (32u * (blk0 + (cnt >> 2)) + lB) + (cnt & 3u);
}


// ---- CTA-cooperative sweep of very long rows (the block-granularity sampler) ----
//
// When a warp meets a row of at least kCoopMinSupers supergroups while other warps of its CTA
// have run out of queries, it posts the row on the CTA's board.  The owner keeps sweeping from
// the front with its usual loop; idle warps draw tickets and take chunks of full interior
// supergroups from the back (ticket k covers the kCoopChunkSupers supergroups below
// end_super - k * kCoopChunkSupers).  At every supergroup boundary the owner looks at the ticket
// count and stops where the helpers' part begins.  Helpers fold their best (key, strip id) into
// the board with one 64-bit atomicMin: the block-level combine.  min over (key, id) is
// order-independent and idempotent, so overlaps are harmless and the walk is bit-identical to the
// single-warp sweep.  Busy warps never help: that was measured and nearly halved the throughput
// of the bulk phase.  Stands in for sampler_block (include/sampler.cuh:87-127) and the block
// phase of the reference scheduler (include/walker.cuh:1397-1419), which stalls the whole CTA on
// one query at a time.
constexpr uint32_t kCoopMinSupers = 16;   // rows from 16 supergroups (about 32,000 edges) may be shared
constexpr uint32_t kCoopChunkSupers = 4;  // supergroups per ticket (32 KB)
constexpr uint32_t kCoopSpinLimit = 1u << 22;
constexpr unsigned int kCoopClosed = 0xFFFF0000u;  // ticket word while no row is posted (epoch 0xFFFF is never used)
constexpr unsigned long long kCoopFailed = 0xFFFFFFFFFFFFFFFEull;

struct CoopTask {
  unsigned int walking;   // warps of the CTA that still have queries of their own
  unsigned int lock;      // 1 while a warp owns the board
  unsigned int open;      // 1 while a row is posted
  unsigned int ticket;    // epoch << 16 | tickets drawn; drawn with atomicAdd
  unsigned int epoch;     // epoch of the posted row, 0 .. 0xFFFE
  unsigned int done;      // tickets served
  unsigned int end_super; // the shared supergroups are [1, end_super), handed out from the back
  unsigned long long best;  // key bits << 32 | strip id, atomicMin
  uint32_t c1, qlo, qhi;
  StepCtx c;              // the row; `from` and `flags` are per helper
};

__device__ __forceinline__ unsigned int ld_volatile(const unsigned int* p) {
  return *reinterpret_cast<const volatile unsigned int*>(p);
}

// Full interior supergroups [s0, s1) of the row c (every sub-block complete, no boundary quad),
// by one warp.  False when a staged copy did not arrive in time.
template <int APP, bool CLEAN>
__device__ __forceinline__ bool sweep_supers(const WalkArgs& a, const StepCtx& c, uint32_t s0, uint32_t s1,
                                             uint32_t lane, uint32_t c1, uint32_t qlo, uint32_t qhi, Ring& ring,
                                             const unsigned char* ring_ptr, Best& best) {
  SuperAcc acc{0.0f, 0.0f, s0 / 3u, s0 % 3u, fw::Philox4{0u, 0u, 0u, 0u}};
  acc.r = fw::philox4x32_10(acc.g * 32u + lane, c1, qlo, qhi, a.k0, a.k1);
  if constexpr (APP == FW_APP_NODE2VEC) {
    const uint32_t b0 = 4u * s0, bend = 4u * s1;
    if (lane == 0) {
#pragma unroll
      for (uint32_t t = 0; t < kStages; ++t)
        if (b0 + t < bend) ring_fill<SweepApp<APP>::value>(c, ring, b0 + t, t);
    }
    uint32_t t = 0;
#pragma unroll 1
    for (uint32_t b = b0; b < bend; ++b) {
      float A;
      if (!ring_sub<SweepApp<APP>::value, CLEAN>(a, c, b, bend, lane, ring, ring_ptr, t, A)) return false;
      t = t + 1u == (uint32_t)kStages ? 0u : t + 1u;
      absorb<APP, CLEAN>(a, c, acc, best, A, b, false, true, lane, c1, qlo, qhi);
    }
  } else {
    if (lane == 0) {
      half_fill(c, ring, 2u * s0);
      half_fill(c, ring, 2u * s0 + 1u);
    }
    const int4* lane_ptr = reinterpret_cast<const int4*>(ring_ptr) + lane;
#pragma unroll 1
    for (uint32_t s = s0; s < s1; ++s) {
      float W;
      if (!super_turn<SweepApp<APP>::value, CLEAN, false>(c, s, 2u * s1, 2u * s1, lane, ring, lane_ptr, W)) return false;
      absorb_super<APP, CLEAN>(a, c, acc, best, W, s, false, lane, c1, qlo, qhi);
    }
  }
  return true;
}

// The out-of-line helpers below receive the kernel arguments by address.  They read the fields
// of a row sweep once into a local copy: every field that sweep_supers, sub_global, absorb,
// n2v_test, n2v_strip_exact or the Philox calls read must be listed here (the rest of the copy is
// never read and costs nothing).
__device__ __forceinline__ WalkArgs sweep_args(const WalkArgs& args) {
  WalkArgs a;
  a.adj = args.adj;
  a.inv_p = args.inv_p;
  a.inv_q = args.inv_q;
  a.n2v_fmax = args.n2v_fmax;  // bound of node2vec's optimistic key (n2v_test)
  a.k0 = args.k0;
  a.k1 = args.k1;
  return a;
}

// An idle warp serves tickets of the posted row until they stop being valid.  Every lane of the
// warp must call it.  Returns the warp's ring parity in bits 1.., and in bit 0 whether all went
// well (0: a staged copy did not arrive).  Out of line: only idle warps run it.
template <int APP, bool CLEAN>
__device__ __noinline__ uint32_t coop_serve(const WalkArgs& args, CoopTask* task, uint32_t lane, Ring ring,
                                            const unsigned char* ring_ptr, uint32_t* my_flags) {
  const WalkArgs a = sweep_args(args);
  for (;;) {
    unsigned int tk = 0, mine = 0;
    if (lane == 0) {
      tk = atomicAdd(&task->ticket, 1u);
      __threadfence_block();
      // a ticket belongs to the row whose epoch it carries; that row stays posted until every
      // ticket drawn from its counter has been served
      mine = (tk >> 16) == ld_volatile(&task->epoch);
    }
    tk = __shfl_sync(0xFFFFFFFFu, tk, 0);
    if (!__shfl_sync(0xFFFFFFFFu, mine, 0)) return (ring.parity << 1) | 1u;
    const uint32_t k = tk & 0xFFFFu;
    const uint32_t end_super = task->end_super;
    const uint32_t below = k * kCoopChunkSupers;
    Best best{0xFFFFFFFFu, 0xFFFFFFFFu, 0u, 0.0f};
    bool fine = true;
    if (below + 1u < end_super) {  // something is left above supergroup 0
      const uint32_t s1 = end_super - below;
      const uint32_t s0 = s1 > kCoopChunkSupers + 1u ? s1 - kCoopChunkSupers : 1u;
      StepCtx c = task->c;
      c.flags = my_flags;
      fine = sweep_supers<APP, CLEAN>(a, c, s0, s1, lane, task->c1, task->qlo, task->qhi, ring, ring_ptr, best);
      warp_argmin(best.key, best.id);
    }
    else __nanosleep(512);  // nothing left above the owner's part: do not hammer the ticket counter
    if (lane == 0) {
      if (fine && best.id != 0xFFFFFFFFu) atomicMin(&task->best, ((unsigned long long)best.key << 32) | best.id);
      __threadfence_block();
      if (fine) atomicAdd(&task->done, 1u);
    }
    if (!fine) return ring.parity << 1;
  }
}

// A warp out of queries: lend a hand if a row is posted.  False when a staged copy did not arrive.
template <int APP, bool CLEAN>
__device__ __forceinline__ bool coop_help(const WalkArgs& a, CoopTask* task, uint32_t lane, Ring& ring,
                                          const unsigned char* ring_ptr, uint32_t* my_flags) {
  unsigned int open = 0;
  if (lane == 0) open = ld_volatile(&task->open);
  if (!__shfl_sync(0xFFFFFFFFu, open, 0)) return true;
  const uint32_t r = coop_serve<APP, CLEAN>(a, task, lane, ring, ring_ptr, my_flags);
  ring.parity = r >> 1;
  return (r & 1u) != 0;
}

// Owner: posts the row when an idle warp exists and the board is free.  Out of line (rare).
__device__ __noinline__ unsigned int coop_post(CoopTask* task, const int4* prim, const int4* sec, uint32_t nq,
                                               uint32_t head, uint32_t tail, int32_t prev, const int32_t* prow,
                                               uint32_t plen, int32_t want, uint32_t c1, uint32_t qlo, uint32_t qhi,
                                               uint32_t end_super, uint32_t lane) {
  unsigned int got = 0;
  if (lane == 0 && ld_volatile(&task->walking) < (unsigned int)kWarpsPerCta && atomicCAS(&task->lock, 0u, 1u) == 0u) {
    got = 1;
    unsigned int ep = ld_volatile(&task->epoch) + 1u;
    if (ep >= 0xFFFFu) ep = 0u;
    StepCtx c;
    c.prim = prim; c.sec = sec; c.nq = nq; c.head = head; c.tail = tail; c.prev = prev;
    c.prow = prow; c.plen = plen; c.want = want; c.from = 0u; c.flags = nullptr;
    task->c = c;
    task->c1 = c1; task->qlo = qlo; task->qhi = qhi;
    task->end_super = end_super;
    task->done = 0u;
    task->best = ~0ull;
    task->epoch = ep;
    __threadfence_block();
    atomicExch(&task->ticket, ep << 16);
    __threadfence_block();
    atomicExch(&task->open, 1u);
  }
  return __shfl_sync(0xFFFFFFFFu, got, 0);
}

// Owner: no more tickets for this row; returns how many were drawn.
__device__ __forceinline__ uint32_t coop_stop_tickets(CoopTask* task, uint32_t lane) {
  unsigned int k = 0;
  if (lane == 0) {
    atomicExch(&task->open, 0u);
    k = atomicExch(&task->ticket, kCoopClosed) & 0xFFFFu;
  }
  return __shfl_sync(0xFFFFFFFFu, k, 0);
}

// Owner: waits (bounded) until the drawn tickets are served, folds the helpers' result into its
// own packed (key, id) and frees the board.  kCoopFailed when the wait ran out.  Out of line.
__device__ __noinline__ unsigned long long coop_close(CoopTask* task, uint32_t tickets, unsigned long long own,
                                                      uint32_t lane) {
  unsigned long long fin = kCoopFailed;
  if (lane == 0) {
    for (uint32_t spin = 0; spin < kCoopSpinLimit; ++spin) {
      if (ld_volatile(&task->done) >= tickets) { fin = own; break; }
      __nanosleep(64);
    }
    __threadfence_block();
    if (fin != kCoopFailed) {
      const unsigned long long theirs = *reinterpret_cast<volatile unsigned long long*>(&task->best);
      if (theirs < fin) fin = theirs;
    }
    __threadfence_block();
    if (fin != kCoopFailed) atomicExch(&task->lock, 0u);  // after a failed wait the board stays taken
  }
  return __shfl_sync(0xFFFFFFFFu, fin, 0);
}

// Owner: total bias and pick word of strip B when another warp reduced it.  Out of line (rare).
// Returns the pick word in the high half and the bits of the total in the low half.
template <int APP, bool CLEAN>
__device__ __noinline__ unsigned long long strip_redo(const WalkArgs& args, StepCtx c, uint32_t B, uint32_t c1,
                                                      uint32_t qlo, uint32_t qhi, uint32_t lane) {
  const WalkArgs a = sweep_args(args);
  const uint32_t sW = B >> 5, lW = B & 31u;
  const uint32_t last_b = (c.nq + fw::kQuadsPerSub - 1) / fw::kQuadsPerSub - 1u;
  const uint32_t pick = fw::philox4x32_10((sW / 3u) * 32u + lW, c1, qlo, qhi, a.k0, a.k1).w;
  float A[4];
#pragma unroll 1
  for (uint32_t i = 0; i < 4u; ++i) {
    const uint32_t b = 4u * sW + i;
    A[i] = 0.0f;
    if (b <= last_b) {  // warp-uniform
      A[i] = sub_global<SweepApp<APP>::value, CLEAN>(a, c, b, lW);
    }
  }
  const float W = __fadd_rn(__fadd_rn(A[0], A[1]), __fadd_rn(A[2], A[3]));
  return ((unsigned long long)pick << 32) | __float_as_uint(W);
}

// The strip sampler of DeepWalk, PPR and MetaPath on a row of more than 32 quads: the whole row
// streams through the warp's two 4 KB stages (see half_take).  `r0`: the lane's first Philox block.
template <int APP, int MODE, bool CLEAN>
__device__ __forceinline__ uint32_t sweep_streamed(const WalkArgs& a, const StepCtx& c, uint32_t c1, uint32_t qlo,
                                                   uint32_t qhi, uint32_t lane, Ring& ring, const unsigned char* ring_ptr,
                                                   CoopTask* task, const fw::Philox4& r0) {
  constexpr int SAPP = SweepApp<APP, MODE>::value;
  Best best{0xFFFFFFFFu, 0xFFFFFFFFu, 0u, 0.0f};
  const uint32_t n_half = (c.nq + kHalfQuads - 1u) / kHalfQuads;
  const uint32_t end_super = ((n_half + 1u) >> 1) - 1u;  // the row's last supergroup
  if (lane == 0) {
    half_fill(c, ring, 0u);
    if (n_half > 1u) half_fill(c, ring, 1u);
  }
  SuperAcc acc{0.0f, 0.0f, 0u, 0u, r0};
  // A very long row is posted for the CTA's idle warps, which take supergroups from the back.
  bool posted = false;
  if (MODE == kModeStripShared && end_super + 1u >= kCoopMinSupers)
    posted = coop_post(task, c.prim, c.sec, c.nq, c.head, c.tail, c.prev, c.prow, c.plen, c.want, c1, qlo, qhi,
                       end_super, lane) != 0u;
  uint32_t tickets = 0;
  bool stopped = false;
  const int4* lane_ptr = reinterpret_cast<const int4*>(ring_ptr) + lane;
  uint32_t sg = 0;
#pragma unroll 1
  for (;;) {
    const bool last = sg == end_super;
    float W;
    bool ok;
    if (sg == 0u || last) ok = super_turn<SAPP, CLEAN, true>(c, sg, n_half, n_half, lane, ring, lane_ptr, W);
    else ok = super_turn<SAPP, CLEAN, false>(c, sg, n_half, n_half, lane, ring, lane_ptr, W);
    if (!ok) { ring.failed = true; return 0xFFFFFFFFu; }
    absorb_super<APP, CLEAN>(a, c, acc, best, W, sg, last, lane, c1, qlo, qhi);
    if (last) break;
    ++sg;
    if (posted && sg < end_super) {
      // this warp stops in front of the supergroups the drawn tickets cover
      unsigned int k = 0;
      if (lane == 0) k = ld_volatile(&task->ticket) & 0xFFFFu;
      if (sg + __shfl_sync(0xFFFFFFFFu, k, 0) * kCoopChunkSupers >= end_super) {
        // hand-over: both halves of supergroup sg are in flight or staged; wait for them, drop
        // them, and go on with the row's last supergroup, which stays with this warp
        tickets = coop_stop_tickets(task, lane);
        stopped = true;
        bool arrived = mbar_wait(ring.bar, ring.parity & 1u);
        arrived = mbar_wait(ring.bar + 8u, (ring.parity >> 1) & 1u) && arrived;
        ring.parity ^= 3u;
        if (!__all_sync(0xFFFFFFFFu, arrived)) { ring.failed = true; return 0xFFFFFFFFu; }
        sg = end_super;
        if (lane == 0) {
          half_fill(c, ring, 2u * sg);
          if (2u * sg + 1u < n_half) half_fill(c, ring, 2u * sg + 1u);
        }
        acc.g = sg / 3u;
        acc.m = sg - 3u * acc.g;
        acc.r = fw::philox4x32_10(acc.g * 32u + lane, c1, qlo, qhi, a.k0, a.k1);
      }
    }
  }
  if (posted && !stopped) tickets = coop_stop_tickets(task, lane);
  warp_argmin(best.key, best.id);
  uint32_t B = best.id;
  if (posted) {
    const unsigned long long own = ((unsigned long long)best.key << 32) | best.id;
    const unsigned long long fin = coop_close(task, tickets, own, lane);
    if (fin == kCoopFailed) { ring.failed = true; return 0xFFFFFFFFu; }
    B = (uint32_t)fin;
    if (B != 0xFFFFFFFFu && fin != own) {  // another warp reduced the winning strip
      const unsigned long long pw = strip_redo<APP, CLEAN>(a, c, B, c1, qlo, qhi, lane);
      return pick_in_row<SAPP, CLEAN>(a, c, B, (uint32_t)(pw >> 32), __uint_as_float((uint32_t)pw), lane);
    }
  }
  if (B == 0xFFFFFFFFu) return B;
  FW_PROF(const long long tp0 = clock64();)
  const uint32_t pick = __shfl_sync(0xFFFFFFFFu, best.pick, (int)(B & 31u));
  const float WB = __shfl_sync(0xFFFFFFFFu, best.W, (int)(B & 31u));
  // a row of one supergroup is still in the ring
  const uint32_t rel = end_super == 0u ? pick_in_row<SAPP, CLEAN, true>(a, c, B, pick, WB, lane, ring_ptr)
                                       : pick_in_row<SAPP, CLEAN>(a, c, B, pick, WB, lane);
  FW_PROF(if (lane == 0) atomicAdd(&g_prof[7], (unsigned long long)(clock64() - tp0));)
  return rel;
}

// One weighted pick in the row described by c, by one warp.  Returns the
// edge index relative to quad 0 of the row, or 0xFFFFFFFF when no edge has
// positive bias.
template <int APP, int MODE, bool CLEAN>
__device__ __forceinline__ uint32_t sample_row_warp(const WalkArgs& a, const StepCtx& c, uint32_t step,
                                                    uint32_t qlo, uint32_t qhi, uint32_t lane, Ring& ring,
                                                    const unsigned char* ring_ptr, CoopTask* task) {
  const uint32_t c1 = step | (fw::kPurposeScan << 28);
  const int4 zero = make_int4(0, 0, 0, 0);
  if (MODE == FW_GROUP_EDGE) {
    uint32_t best_key = 0xFFFFFFFFu, best_id = 0xFFFFFFFFu;
    for (uint32_t base = 0; base < c.nq; base += 32) {  // warp-uniform trip count
      const uint32_t q = base + lane;
      const bool valid = q < c.nq;
      const int4 raw = valid ? __ldg(c.prim + q) : zero;
      const int4 nb = (APP == FW_APP_NODE2VEC && valid) ? __ldg(c.sec + q) : zero;
      uint32_t linked = 0u;
      if (APP == FW_APP_NODE2VEC && c.prev >= 0) linked = n2v_linked(a, c, nb, q, true, lane);
      float4 v = quad_bias<APP, CLEAN>(a, c, raw, nb, q, linked);
      mask_quad(v, q, c.head, c.tail);
      const fw::Philox4 r = fw::philox4x32_10(q, c1, qlo, qhi, a.rk);
      const float vs[4] = {v.x, v.y, v.z, v.w};
      const uint32_t rs[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (vs[k] > 0.0f) {
          const uint32_t bits = __float_as_uint(__fdiv_rn(fw::exp_key(rs[k]), vs[k]));
          if (bits < best_key) { best_key = bits; best_id = 4u * q + k; }
        }
      }
    }
    warp_argmin(best_key, best_id);
    return best_id;
  }

  // ---- strips ----
  // Strip (s,l): the 16 quads 512 s + 32 j + l.  Philox block g of lane l (counter word
  // 0 = g*32 + l) serves supergroups 3g, 3g+1, 3g+2 (words 0..2 -> keys) and carries in
  // word 3 the uniform for the in-strip pick.
  Best best{0xFFFFFFFFu, 0xFFFFFFFFu, 0u, 0.0f};
  // round keys straight from the kernel arguments; the node2vec kernels, short of registers,
  // measured faster with the key schedule computed in place
  fw::Philox4 r = APP == FW_APP_NODE2VEC ? fw::philox4x32_10(lane, c1, qlo, qhi, a.k0, a.k1)
                                         : fw::philox4x32_10(lane, c1, qlo, qhi, a.rk);

  if (c.nq <= 32u) {
    // Short row: one quad per lane, strip = that quad; the winner's quad travels by shuffle.
    float4 v = load_quad<APP, CLEAN>(a, c, lane, true);
    offer(best, r.x, r.w, sum4(v), lane);
    warp_argmin(best.key, best.id);
    if (best.id == 0xFFFFFFFFu) return best.id;
    const int src = (int)best.id;
    v.x = __shfl_sync(0xFFFFFFFFu, v.x, src);
    v.y = __shfl_sync(0xFFFFFFFFu, v.y, src);
    v.z = __shfl_sync(0xFFFFFFFFu, v.z, src);
    v.w = __shfl_sync(0xFFFFFFFFu, v.w, src);
    const uint32_t pick = __shfl_sync(0xFFFFFFFFu, r.w, src);
    const float thr = __fmul_rn((float)(pick >> 8) * 0x1p-24f, sum4(v));
    const float p0 = v.x, p1 = __fadd_rn(p0, v.y), p2 = __fadd_rn(p1, v.z), p3 = __fadd_rn(p2, v.w);
    uint32_t cnt = (p0 <= thr ? 1u : 0u) + (p1 <= thr ? 1u : 0u) + (p2 <= thr ? 1u : 0u) + (p3 <= thr ? 1u : 0u);
    if (cnt >= 4u) cnt = v.w > 0.0f ? 3u : v.z > 0.0f ? 2u : v.y > 0.0f ? 1u : 0u;
    return 4u * (uint32_t)src + cnt;
  }

  if constexpr (APP != FW_APP_NODE2VEC) return sweep_streamed<APP, MODE, CLEAN>(a, c, c1, qlo, qhi, lane, ring, ring_ptr, task, r);

  // node2vec.  The row is swept in sub-blocks of 128 quads (2 KB): the first and the last straight
  // from global memory (boundary quads, partial fill), the interior ones through a ring of two
  // 2 KB stages when there are any.  Four sub-blocks make a supergroup; a lane's four partial
  // sums A0..A3 are combined as (A0+A1)+(A2+A3) and tested once per supergroup.
  const uint32_t nb = (c.nq + fw::kQuadsPerSub - 1) / fw::kQuadsPerSub;
  const uint32_t last_b = nb - 1u;
  const bool ringed = nb >= 3u;
  if (ringed && lane == 0) {
#pragma unroll
    for (uint32_t t = 0; t < kStages; ++t)
      if (1u + t < last_b) ring_fill<SweepApp<APP, MODE>::value>(c, ring, 1u + t, t);
  }
  SuperAcc acc{0.0f, 0.0f, 0u, 0u, r};
  // A very long row is posted for the CTA's idle warps, which take supergroups from the back.
  const uint32_t end_super = ((nb + 3u) >> 2) - 1u;  // the last supergroup stays with this warp
  bool posted = false;
  if (MODE == kModeStripShared && nb > 4u * (kCoopMinSupers - 1u))
    posted = coop_post(task, c.prim, c.sec, c.nq, c.head, c.tail, c.prev, c.prow, c.plen, c.want, c1, qlo, qhi,
                       end_super, lane) != 0u;
  // this warp stops in front of the supergroups the drawn tickets cover
  auto taken = [&](uint32_t b) {
    unsigned int k = 0;
    if (lane == 0) k = ld_volatile(&task->ticket) & 0xFFFFu;
    return (b >> 2) + __shfl_sync(0xFFFFFFFFu, k, 0) * kCoopChunkSupers >= end_super;
  };
  absorb<APP, CLEAN>(a, c, acc, best, sub_first<SweepApp<APP, MODE>::value, CLEAN>(a, c, nb > 1u, lane), 0u, nb == 1u, false, lane, c1, qlo, qhi);
  uint32_t b = 1;
  if (!ringed) {
#pragma unroll 1
    for (; b < last_b; ++b) {
      if (posted && (b & 3u) == 0u && taken(b)) break;
      absorb<APP, CLEAN>(a, c, acc, best, sub_global<SweepApp<APP, MODE>::value, CLEAN>(a, c, b, lane), b, false, true, lane, c1, qlo, qhi);
    }
  } else {
    uint32_t t = 0;
    // Kept rolled on purpose: an unrolled sweep measured slower (instruction cache shared by the
    // warps of an SM, which sit at different places of the kernel), and node2vec's key test is
    // large: a second copy of it in a leaner loop cost more than the loop saved (157 against
    // 107 ms on R-MAT scale 20, edge factor 32).
#pragma unroll 1
    for (; b < last_b; ++b) {
      if (posted && (b & 3u) == 0u && taken(b)) {
        // hand-over: the copies already in flight for b, b+1, .. are waited for and dropped
        bool ok = true;
        for (uint32_t i = 0; i < (uint32_t)kStages && b + i < last_b; ++i) {
          const uint32_t st = (t + i) % (uint32_t)kStages;
          ok = mbar_wait(ring.bar + 8u * st, (ring.parity >> st) & 1u) && ok;
          ring.parity ^= 1u << st;
        }
        if (!__all_sync(0xFFFFFFFFu, ok)) { ring.failed = true; return 0xFFFFFFFFu; }
        break;
      }
      float A;
      if (!ring_sub<SweepApp<APP, MODE>::value, CLEAN>(a, c, b, last_b, lane, ring, ring_ptr, t, A)) {
        ring.failed = true;
        return 0xFFFFFFFFu;
      }
      absorb<APP, CLEAN>(a, c, acc, best, A, b, false, true, lane, c1, qlo, qhi);
      t = t + 1u == (uint32_t)kStages ? 0u : t + 1u;
    }
  }
  uint32_t tickets = 0;
  if (posted) {
    tickets = coop_stop_tickets(task, lane);
    if (b < last_b) {
      // stopped early: the last supergroup (partial fill, row end) is still this warp's
      acc.g = end_super / 3u;
      acc.m = end_super - 3u * acc.g;
      acc.r = fw::philox4x32_10(acc.g * 32u + lane, c1, qlo, qhi, a.k0, a.k1);
#pragma unroll 1
      for (b = 4u * end_super; b < last_b; ++b)
        absorb<APP, CLEAN>(a, c, acc, best, sub_global<SweepApp<APP, MODE>::value, CLEAN>(a, c, b, lane), b, false, false, lane, c1, qlo, qhi);
    }
  }
  if (nb > 1u) absorb<APP, CLEAN>(a, c, acc, best, sub_global<SweepApp<APP, MODE>::value, CLEAN>(a, c, last_b, lane), last_b, true, false, lane, c1, qlo, qhi);
  warp_argmin(best.key, best.id);
  uint32_t B = best.id;
  if (posted) {
    const unsigned long long own = ((unsigned long long)best.key << 32) | best.id;
    const unsigned long long fin = coop_close(task, tickets, own, lane);
    if (fin == kCoopFailed) { ring.failed = true; return 0xFFFFFFFFu; }
    B = (uint32_t)fin;
    if (B != 0xFFFFFFFFu && fin != own) {  // another warp reduced the winning strip
      const unsigned long long pw = strip_redo<APP, CLEAN>(a, c, B, c1, qlo, qhi, lane);
      if (APP == FW_APP_NODE2VEC && c.prev >= 0) return n2v_pick<CLEAN>(a, c, B, (uint32_t)(pw >> 32), lane);
      return pick_in_row<SweepApp<APP, MODE>::value, CLEAN>(a, c, B, (uint32_t)(pw >> 32), __uint_as_float((uint32_t)pw), lane);
    }
  }
  if (B == 0xFFFFFFFFu) return B;
  if (APP == FW_APP_NODE2VEC && c.prev >= 0)
    return n2v_pick<CLEAN>(a, c, B, __shfl_sync(0xFFFFFFFFu, best.pick, (int)(B & 31u)), lane);
  return pick_in_row<SweepApp<APP, MODE>::value, CLEAN>(a, c, B, __shfl_sync(0xFFFFFFFFu, best.pick, (int)(B & 31u)),
                                                  __shfl_sync(0xFFFFFFFFu, best.W, (int)(B & 31u)), lane);
}

template <int APP, int MODE, bool CLEAN, typename OffT>
constexpr int min_blocks() {
  // Resident CTAs of 256 threads per SM the register allocation is held to (65,536 registers:
  // 3 CTAs -> 85 per thread, 4 -> 64, 5 -> 48).  The strip kernels of DeepWalk, PPR and MetaPath
  // hold 8 KB of staging ring per warp, so three CTAs per SM is what shared memory allows as well.
  return MODE == FW_GROUP_EDGE ? 2 : APP == FW_APP_NODE2VEC ? FW_N2V_MIN_BLOCKS : FW_MIN_BLOCKS;
}

// The strip sampler on a row of at most SQ quads (one stage: every row that is not a hub's)
// that was staged ahead into stage T of the warp's ring: the copy of the next slot's row is in
// flight while this one is reduced.  Same strips, keys and pick as sample_row_warp.
template <int APP, bool CLEAN, uint32_t SQ>
__device__ __forceinline__ uint32_t sample_staged(const WalkArgs& a, const StepCtx& c, uint32_t step, uint32_t qlo,
                                                  uint32_t qhi, uint32_t lane, Ring& ring, const unsigned char* ring_ptr,
                                                  uint32_t T) {
  const uint32_t c1 = step | (fw::kPurposeScan << 28);
  const fw::Philox4 r = fw::philox4x32_10(lane, c1, qlo, qhi, a.rk);
  const uint32_t ok = mbar_wait_inline(ring.bar + 8u * T, (ring.parity >> T) & 1u);
  ring.parity ^= 1u << T;
  if (!__all_sync(0xFFFFFFFFu, ok != 0u)) { ring.failed = true; return 0xFFFFFFFFu; }
  const unsigned char* stage = ring_ptr + T * (16u * SQ);
  const int4* st = reinterpret_cast<const int4*>(stage) + lane;
  Best best{0xFFFFFFFFu, 0xFFFFFFFFu, 0u, 0.0f};
  if (c.nq <= 32u) {
    // one quad per lane, strip = that quad; the winner's quad travels by shuffle
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (lane < c.nq) {
      v = plain_bias<APP, CLEAN>(st[0], c.want);
      mask_quad(v, lane, c.head, c.tail);
    }
    offer(best, r.x, r.w, sum4(v), lane);
    warp_argmin(best.key, best.id);
    if (best.id == 0xFFFFFFFFu) return best.id;
    const int src = (int)best.id;
    v.x = __shfl_sync(0xFFFFFFFFu, v.x, src);
    v.y = __shfl_sync(0xFFFFFFFFu, v.y, src);
    v.z = __shfl_sync(0xFFFFFFFFu, v.z, src);
    v.w = __shfl_sync(0xFFFFFFFFu, v.w, src);
    const uint32_t pick = __shfl_sync(0xFFFFFFFFu, r.w, src);
    const float thr = __fmul_rn((float)(pick >> 8) * 0x1p-24f, sum4(v));
    const float p0 = v.x, p1 = __fadd_rn(p0, v.y), p2 = __fadd_rn(p1, v.z), p3 = __fadd_rn(p2, v.w);
    uint32_t cnt = (p0 <= thr ? 1u : 0u) + (p1 <= thr ? 1u : 0u) + (p2 <= thr ? 1u : 0u) + (p3 <= thr ? 1u : 0u);
    if (cnt >= 4u) cnt = v.w > 0.0f ? 3u : v.z > 0.0f ? 2u : v.y > 0.0f ? 1u : 0u;
    return 4u * (uint32_t)src + cnt;
  }
  // strip l = quads 32 j + l, j < 8: sub-blocks 0 and 1 of supergroup 0 (the others are empty, and
  // adding their zeros leaves (A0+A1)+(A2+A3) = A0+A1 bit for bit).  Quads past the row, stale
  // bytes of the stage included, are masked.
  float S[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float4 v = plain_bias<APP, CLEAN>(st[32 * j], c.want);
    mask_quad(v, 32u * j + lane, c.head, c.tail);
    S[j] = sum4(v);
  }
  float W = sum_strip(S);
  if (SQ > (uint32_t)fw::kQuadsPerSub && c.nq > (uint32_t)fw::kQuadsPerSub) {  // warp-uniform
#pragma unroll
    for (int j = 4; j < 8; ++j) {
      float4 v = plain_bias<APP, CLEAN>(st[32 * j], c.want);
      mask_quad(v, 32u * j + lane, c.head, c.tail);
      S[j] = sum4(v);
    }
    W = __fadd_rn(W, sum_strip(S + 4));
  }
  offer(best, r.x, r.w, W, lane);
  warp_argmin(best.key, best.id);
  const uint32_t B = best.id;
  if (B == 0xFFFFFFFFu) return B;
  return pick_in_row<APP, CLEAN, true>(a, c, B, __shfl_sync(0xFFFFFFFFu, best.pick, (int)B),
                                       __shfl_sync(0xFFFFFFFFu, best.W, (int)B), lane, stage);
}

// The row of c (at most SQ quads) into stage T (lane 0 only calls this).
template <uint32_t SQ>
__device__ __forceinline__ void row_fill(const StepCtx& c, const Ring& ring, uint32_t T) {
  mbar_expect_tx(ring.bar + 8u * T, 16u * c.nq);
  bulk_g2s(ring.data + T * (16u * SQ), c.prim, 16u * c.nq, ring.bar + 8u * T);
}

// Index of hub vertex v in the ascending list ids[0, n) (v is known to be in it).
__device__ __forceinline__ int32_t hub_index(const int32_t* __restrict__ ids, int32_t n, int32_t v) {
  int32_t lo = 0, hi = n;
  while (lo < hi) {
    const int32_t mid = (lo + hi) >> 1;
    if (__ldg(ids + mid) < v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// One slot each of a list for the lanes that call this together: one atomic for all of them.
__device__ __forceinline__ uint32_t claim_slot(uint32_t* counter) {
  const uint32_t act = __activemask(), lane = threadIdx.x & 31u;
  const int leader = __ffs((int)act) - 1;
  uint32_t first = 0;
  if ((int)lane == leader) first = atomicAdd(counter, (uint32_t)__popc(act));
  return __shfl_sync(act, first, leader) + (uint32_t)__popc(act & ((1u << lane) - 1u));
}

// A walker that arrived at a hub vertex `cur` after k steps waits there for the next hub launch.
__device__ __forceinline__ void hub_park(const HubArgs& hb, long long qi, int32_t k, int32_t cur) {
  const int32_t h = hub_index(hb.hub_ids, hb.n_hubs, cur) * hb.classes + (hb.classes > 1 ? k % hb.classes : 0);
  const uint32_t pos = claim_slot(hb.park_n);
  hb.park_hub[pos] = h;
  hb.park_qi[pos] = (int32_t)qi;
  hb.kstate[qi] = k;
  atomicAdd(hb.hub_cnt + h, 1u);
}

// HUBS: the launch is one of a series (see hub_kernel).  Walkers stop when they arrive at a hub
// vertex and are parked for the next hub launch; the queries of the launch are either all the
// fresh ones or the list the last hub launch left (walkers that went on from a hub to a vertex
// that is not one).
// The tail of the series (HUBS == kHubTail): when few walkers are left parked, batches would be
// nearly empty; one launch then walks them to the end, every walker sweeping for itself.
constexpr int kHubOff = 0, kHubPark = 1, kHubTail = 2, kHubParkLow = 3;  // kHubPark: the limit of 1,016; kHubParkLow: of 504
__host__ __device__ constexpr bool hub_parks(int hubs) { return hubs == kHubPark || hubs == kHubParkLow; }
__host__ __device__ constexpr uint32_t hub_staged_quads(int hubs) { return staged_quads(hubs == kHubParkLow ? kHubLimitLow : kHubLimitHigh); }
template <int APP, int MODE, bool CLEAN, typename OffT, int HUBS>
constexpr int walk_min_blocks() {
  return APP == FW_APP_NODE2VEC ? min_blocks<APP, MODE, CLEAN, OffT>()
       : HUBS == kHubParkLow ? 4 : HUBS == kHubPark ? 3 : min_blocks<APP, MODE, CLEAN, OffT>();
}
template <int APP, int MODE, bool CLEAN, typename OffT, int HUBS = kHubOff>
__global__ void __launch_bounds__(kThreads, walk_min_blocks<APP, MODE, CLEAN, OffT, HUBS>()) walk_kernel(const __grid_constant__ WalkArgs a) {
  extern __shared__ __align__(128) unsigned char s_dyn[];
  __shared__ __align__(8) unsigned long long s_bar[kWarpsPerCta][kStages];
  __shared__ uint32_t s_flags[APP == FW_APP_NODE2VEC ? kWarpsPerCta : 1][32];  // node2vec match flags
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  constexpr uint32_t kStagedQuads = hub_staged_quads(HUBS);
  constexpr uint32_t kRingPerWarp = MODE == FW_GROUP_EDGE ? 0u
                                  : (hub_parks(HUBS) && APP != FW_APP_NODE2VEC) ? 2u * 16u * kStagedQuads : ring_bytes<APP>();
  uint32_t* s_hist = reinterpret_cast<uint32_t*>(s_dyn + kRingPerWarp * kWarpsPerCta);
  const unsigned char* ring_ptr = s_dyn + kRingPerWarp * warp;
  Ring ring;
  ring.data = smem_addr(ring_ptr);
  ring.bar = smem_addr(&s_bar[warp][0]);
  ring.parity = 0u;
  ring.failed = false;
  if (MODE != FW_GROUP_EDGE && lane == 0) {
#pragma unroll
    for (int t = 0; t < kStages; ++t) mbar_init(ring.bar + 8u * t, 1u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __shared__ CoopTask s_task;  // the CTA's board for rows shared between its warps
  if (threadIdx.x == 0) {
    s_task.walking = kWarpsPerCta; s_task.lock = 0u; s_task.open = 0u; s_task.ticket = kCoopClosed;
    s_task.epoch = 0u; s_task.done = 0u; s_task.end_super = 0u; s_task.best = ~0ull;
  }
  if (a.hist_in_smem)
    for (int z = threadIdx.x; z <= a.d; z += blockDim.x) s_hist[z] = 0u;
  __syncthreads();

  const OffT* __restrict__ xadj = static_cast<const OffT*>(a.xadj);
  const int64_t D = (int64_t)a.d + 1;
  const int4* const prim_base = reinterpret_cast<const int4*>(APP == FW_APP_METAPATH ? (const void*)a.label
                                                                                     : (const void*)a.weight);
  const int4* const sec_base = reinterpret_cast<const int4*>(a.adj);
  unsigned long long my_steps = 0, my_scanned = 0;
  uint32_t status = 0;

  // A warp keeps kSlots queries in flight.  The state of slot i (the role of the reference's Task,
  // include/gpu_task.cuh:24-78) lives in the registers of lane i, so everything that is one
  // dependent memory access per query -- the start vertex, the row bounds of the current vertex,
  // the chosen neighbour, the result cell, the stop test -- is issued for all slots by one
  // instruction and the round trips of the slots overlap.  Only the weighted pick itself takes
  // the whole warp, one slot after the other.
  constexpr uint32_t kNone = 0xFFFFFFFFu;
  constexpr int kSlots = slots_of<APP>();
  constexpr int kClaim = 2 * kSlots > kMinClaim ? 2 * kSlots : kMinClaim;  // queries claimed per atomic
  const bool slot_lane = lane < (uint32_t)kSlots;
  long long qi = -1;                 // index of the slot's query in this launch
  uint32_t qlo = 0, qhi = 0;         // its global id (key of the random stream)
  int32_t cur = 0, prev = -1, k = 0; // current and previous vertex, steps taken
  OffT rb = 0, pb = 0;               // first edge of the current and of the previous vertex's row
  uint32_t rlen = 0, plen = 0;       // their lengths
  uint32_t st = 0;                   // 0: empty, 1: walking, 2: walk over, to be closed
  uint32_t my_rel = kNone;           // the pick of this round
  long long res_next = 0, res_end = 0;  // queries claimed by the warp and not yet handed to a slot
  bool exhausted = false;

  unsigned long long* const work = HUBS != kHubOff ? a.hub.work : a.scratch + kSlotCounter;
  const long long n_work = (HUBS != kHubOff && a.hub.list != nullptr) ? (long long)*a.hub.list_n : (long long)a.n;
  FW_PROF(unsigned long long prof_t[3] = {0, 0, 0}, prof_n[3] = {0, 0, 0}, prof_sub = 0; const long long prof_begin = clock64();)
  if constexpr (kSlots == 1) {
    // One query per warp, walked to its end (or, in a hub-batched series, to the next hub) with all
    // state in uniform registers (node2vec: its kernels are the largest, and the slot bookkeeping
    // below cost them a third of their speed).
    const bool resumed = HUBS != kHubOff && a.hub.list != nullptr;
    while (!ring.failed) {
      long long first = 0;
      if (lane == 0) first = (long long)atomicAdd(work, (unsigned long long)kMinClaim);
      first = __shfl_sync(0xFFFFFFFFu, first, 0);
      if (first >= n_work) break;
      const long long stop = first + kMinClaim < n_work ? first + kMinClaim : n_work;
      for (long long idx = first; idx < stop && !ring.failed; ++idx) {
        const long long q1 = resumed ? (long long)__ldg(a.hub.list + idx) : idx;
        const uint64_t qid = a.qid_base + (uint64_t)q1 * a.qid_stride;
        const uint32_t ql = (uint32_t)qid, qh = (uint32_t)(qid >> 32);
        int32_t* __restrict__ row_out = a.result + q1 * D;
        StepCtx c;
        c.prev = -1; c.prow = a.adj; c.plen = 0u; c.want = 0; c.from = 0u;
        c.flags = &s_flags[APP == FW_APP_NODE2VEC ? warp : 0][0];
        int kk = 0;
        int32_t at;
        if (resumed) {  // a walker a hub launch moved on: position and previous vertex from the table
          kk = a.hub.kstate[q1];
          at = row_out[kk];
          if (kk > 0) {
            c.prev = row_out[kk - 1];
            const int64_t pb0 = (int64_t)__ldg(xadj + c.prev);
            c.prow = a.adj + pb0;
            c.plen = (uint32_t)((int64_t)__ldg(xadj + c.prev + 1) - pb0);
          }
        } else {
          at = __ldg(a.starts + q1);
          if (lane == 0) row_out[0] = at;
        }
        bool parked = false;
        if (at < 0 || (int64_t)at >= a.V) {
          status |= FW_STATUS_BAD_START;
        } else {
          while (kk < a.d) {
            const int64_t b = (int64_t)__ldg(xadj + at), e = (int64_t)__ldg(xadj + at + 1);
            if (e <= b) break;
            if (hub_parks(HUBS) && (uint64_t)(e - b) >= (uint64_t)a.hub.min_degree) {
              if (lane == 0) hub_park(a.hub, q1, kk, at);  // the hub launch takes the walker from here
              parked = true;
              break;
            }
            const int64_t q0 = b >> 2;
            c.prim = prim_base + q0;
            c.sec = sec_base + q0;
            c.nq = (uint32_t)(((e + 3) >> 2) - q0);
            c.head = (uint32_t)(b - 4 * q0);
            c.tail = (uint32_t)(e - 4 * q0);
            if (APP == FW_APP_METAPATH) c.want = a.schema[kk % a.schema_len];
            c.from = 0u;
            const uint32_t rel = sample_row_warp<APP, MODE, CLEAN>(a, c, (uint32_t)kk, ql, qh, lane, ring, ring_ptr, &s_task);
            if (rel == 0xFFFFFFFFu) break;  // include/walker.cuh:1373-1374 (or a failed wait)
            const int32_t nxt = __ldg(a.adj + (4 * q0 + (int64_t)rel));
            if (nxt < 0 || (int64_t)nxt >= a.V) { status |= FW_STATUS_BAD_NEIGHBOR; break; }
            if (lane == 0) row_out[kk + 1] = nxt;  // include/walker.cuh:1380-1381
            my_scanned += (unsigned long long)(e - b);
            c.prev = at; c.prow = a.adj + b; c.plen = (uint32_t)(e - b);  // include/gpu_task.cuh:70-77
            at = nxt;
            ++kk;
            if (APP == FW_APP_PPR) {  // include/app.cuh:88-94
              const fw::Philox4 r = fw::philox4x32_10(0u, (uint32_t)(kk - 1) | (fw::kPurposeStop << 28), ql, qh, a.rk);
              if (r.x < a.tp_thresh) break;
            }
          }
        }
        if (parked) continue;
        for (int z = kk + 1 + (int)lane; z <= a.d; z += 32) row_out[z] = -1;
        my_steps += (unsigned long long)kk;
        if (lane == 0) {
          if (a.hist_in_smem) atomicAdd(&s_hist[kk], 1u);
          else atomicAdd(a.scratch + kSlotHist + kk, 1ull);
          if (HUBS != kHubOff && a.hub.fin) a.hub.fin[q1] = a.hub.fin_tag;
        }
      }
    }
  } else
  while (!ring.failed) {
    // ---- hand queries to the empty slots ----
    const uint32_t empty = __ballot_sync(0xFFFFFFFFu, slot_lane && st == 0u);
    if (empty != 0u && !exhausted) {
      if (res_next >= res_end) {
        long long first = 0;
        if (lane == 0) first = (long long)atomicAdd(work, (unsigned long long)kClaim);
        first = __shfl_sync(0xFFFFFFFFu, first, 0);
        if (first >= n_work) {
          exhausted = true;
        } else {
          res_next = first;
          res_end = first + kClaim < n_work ? first + kClaim : n_work;
        }
      }
      if (!exhausted) {
        const long long mine = res_next + (long long)__popc(empty & ((1u << lane) - 1u));
        if (slot_lane && st == 0u && mine < res_end) {
          const bool resumed = HUBS != kHubOff && a.hub.list != nullptr;
          qi = resumed ? (long long)__ldg(a.hub.list + mine) : mine;
          const uint64_t qid = a.qid_base + (uint64_t)qi * a.qid_stride;
          qlo = (uint32_t)qid;
          qhi = (uint32_t)(qid >> 32);
          prev = -1; pb = 0; plen = 0;
          if (resumed) {  // a walker the last hub launch moved on: its state is what the table holds
            k = a.hub.kstate[qi];
            cur = a.result[qi * D + k];
            st = 1u;
          } else {
            cur = __ldg(a.starts + qi);
            a.result[qi * D] = cur;
            k = 0;
            st = a.d > 0 ? 1u : 2u;
            if (cur < 0 || (int64_t)cur >= a.V) { status |= FW_STATUS_BAD_START; st = 2u; }
          }
        }
        res_next += (long long)__popc(empty);
        if (res_next > res_end) res_next = res_end;
      }
    }
    if (__ballot_sync(0xFFFFFFFFu, st != 0u) == 0u) {
      if (exhausted) break;
      continue;
    }
    // ---- row bounds of every walking slot ----
    if (st == 1u) {
      const OffT b = __ldg(xadj + cur), e = __ldg(xadj + cur + 1);
      rb = b;
      rlen = e > b ? (uint32_t)(e - b) : 0u;
      if (rlen == 0u) {
        st = 2u;  // dead end
      } else if (hub_parks(HUBS) && rlen >= a.hub.min_degree) {
        hub_park(a.hub, qi, k, cur);  // the slot is free again; the hub launch takes the walker from here
        st = 0u;
      }
    }
    // ---- the weighted pick: the whole warp on one slot's row at a time ----
    if constexpr (hub_parks(HUBS)) {
      // Every row here is shorter than a hub's: one 4 KB stage holds it.  The two stages take
      // turns, so the next slot's row is on its way while this slot's is reduced.
      uint32_t m = __ballot_sync(0xFFFFFFFFu, st == 1u);
      if (m != 0u) {
        auto slot_ctx = [&](int s, StepCtx& c, uint32_t& ks, uint32_t& ql, uint32_t& qh) {
          const int64_t b = (int64_t)__shfl_sync(0xFFFFFFFFu, rb, s);
          const uint32_t len = __shfl_sync(0xFFFFFFFFu, rlen, s);
          ks = (uint32_t)__shfl_sync(0xFFFFFFFFu, k, s);
          ql = __shfl_sync(0xFFFFFFFFu, qlo, s);
          qh = __shfl_sync(0xFFFFFFFFu, qhi, s);
          const int64_t q0 = b >> 2;
          c.prim = prim_base + q0;
          c.sec = sec_base + q0;
          c.head = (uint32_t)(b - 4 * q0);
          c.tail = c.head + len;
          c.nq = (c.tail + 3u) >> 2;
          c.prev = -1; c.prow = a.adj; c.plen = 0u; c.from = 0u; c.flags = nullptr;
          c.want = APP == FW_APP_METAPATH ? a.schema[ks % (uint32_t)a.schema_len] : 0;
        };
        int s = __ffs((int)m) - 1;
        m &= m - 1u;
        StepCtx c;
        uint32_t ks, ql, qh, T = 0u;
        slot_ctx(s, c, ks, ql, qh);
        if (lane == 0) row_fill<kStagedQuads>(c, ring, T);
        for (;;) {
          int s2 = -1;
          StepCtx c2;
          uint32_t ks2 = 0, ql2 = 0, qh2 = 0;
          if (m != 0u) {
            s2 = __ffs((int)m) - 1;
            m &= m - 1u;
            slot_ctx(s2, c2, ks2, ql2, qh2);
            if (lane == 0) row_fill<kStagedQuads>(c2, ring, T ^ 1u);
          }
          const uint32_t rel = sample_staged<APP, CLEAN, kStagedQuads>(a, c, ks, ql, qh, lane, ring, ring_ptr, T);
          if (ring.failed) break;
          if ((int)lane == s) my_rel = rel;
          if (s2 < 0) break;
          s = s2; c = c2; ks = ks2; ql = ql2; qh = qh2;
          T ^= 1u;
        }
      }
    } else
    for (uint32_t m = __ballot_sync(0xFFFFFFFFu, st == 1u); m != 0u; m &= m - 1u) {
      const int s = __ffs((int)m) - 1;
      const int64_t b = (int64_t)__shfl_sync(0xFFFFFFFFu, rb, s);
      const uint32_t len = __shfl_sync(0xFFFFFFFFu, rlen, s);
      const uint32_t ks = (uint32_t)__shfl_sync(0xFFFFFFFFu, k, s);
      const uint32_t ql = __shfl_sync(0xFFFFFFFFu, qlo, s), qh = __shfl_sync(0xFFFFFFFFu, qhi, s);
      const int64_t q0 = b >> 2;
      StepCtx c;
      c.prim = prim_base + q0;
      c.sec = sec_base + q0;
      c.head = (uint32_t)(b - 4 * q0);
      c.tail = c.head + len;
      c.nq = (c.tail + 3u) >> 2;
      c.prev = -1; c.prow = a.adj; c.plen = 0u; c.want = 0;
      if (APP == FW_APP_NODE2VEC) {
        c.prev = __shfl_sync(0xFFFFFFFFu, prev, s);
        c.prow = a.adj + (int64_t)__shfl_sync(0xFFFFFFFFu, pb, s);
        c.plen = __shfl_sync(0xFFFFFFFFu, plen, s);
      }
      if (APP == FW_APP_METAPATH) c.want = a.schema[ks % (uint32_t)a.schema_len];
      c.from = 0u;
      c.flags = &s_flags[APP == FW_APP_NODE2VEC ? warp : 0][0];
      FW_PROF(const long long ts0 = clock64();)
      const uint32_t rel = sample_row_warp<APP, MODE, CLEAN>(a, c, ks, ql, qh, lane, ring, ring_ptr, &s_task);
      FW_PROF(const long long ts1 = clock64(); const int cls = c.nq <= 32u ? 0 : c.nq <= 2u * fw::kQuadsPerSub ? 1 : 2;
              prof_t[cls] += (unsigned long long)(ts1 - ts0); prof_n[cls] += 1ull;
              if (cls == 2) prof_sub += (c.nq + fw::kQuadsPerSub - 1) / fw::kQuadsPerSub;)
      if (ring.failed) break;
      if ((int)lane == s) my_rel = rel;
    }
    if (ring.failed) break;
    // ---- every walking slot takes its step ----
    if (st == 1u) {
      if (my_rel == kNone) {
        st = 2u;  // no edge with a positive bias: include/walker.cuh:1373-1374
      } else {
        const int32_t nxt = __ldg(a.adj + (4 * ((int64_t)rb >> 2) + (int64_t)my_rel));
        if (nxt < 0 || (int64_t)nxt >= a.V) {
          status |= FW_STATUS_BAD_NEIGHBOR;
          st = 2u;
        } else {
          a.result[qi * D + k + 1] = nxt;  // include/walker.cuh:1380-1381
          my_scanned += (unsigned long long)rlen;
          prev = cur; pb = rb; plen = rlen;  // include/gpu_task.cuh:70-77
          cur = nxt;
          ++k;
          bool stop = k >= a.d;
          if (APP == FW_APP_PPR) {  // include/app.cuh:88-94
            const fw::Philox4 r = fw::philox4x32_10(0u, (uint32_t)(k - 1) | (fw::kPurposeStop << 28), qlo, qhi, a.rk);
            stop = stop || r.x < a.tp_thresh;
          }
          if (stop) st = 2u;
        }
      }
    }
    // ---- close the walks that ended: -1 padding by the whole warp, counters by the slot's lane ----
    for (uint32_t m = __ballot_sync(0xFFFFFFFFu, st == 2u); m != 0u; m &= m - 1u) {
      const int s = __ffs((int)m) - 1;
      const long long qs = __shfl_sync(0xFFFFFFFFu, qi, s);
      const int ks = __shfl_sync(0xFFFFFFFFu, k, s);
      int32_t* __restrict__ row_out = a.result + qs * D;
      for (int z = ks + 1 + (int)lane; z <= a.d; z += 32) row_out[z] = -1;
    }
    if (st == 2u) {
      my_steps += (unsigned long long)k;
      if (a.hist_in_smem) atomicAdd(&s_hist[k], 1u);
      else atomicAdd(a.scratch + kSlotHist + k, 1ull);
      if (HUBS != kHubOff && a.hub.fin) a.hub.fin[qi] = a.hub.fin_tag;
      st = 0u;
    }
  }
  FW_PROF(if (lane == 0) {
    const unsigned long long life = (unsigned long long)(clock64() - prof_begin);
    for (int i = 0; i < 3; ++i) { atomicAdd(&g_prof[i], prof_t[i]); atomicAdd(&g_prof[3 + i], prof_n[i]); }
    atomicAdd(&g_prof[6], prof_sub);
    atomicAdd(&g_prof[8], life - prof_t[0] - prof_t[1] - prof_t[2]);
    atomicAdd(&g_prof[9], life);
  })
  // Out of queries: lend a hand to the rows the CTA's other warps post until all of them are done.
  if (MODE == kModeStripShared) {
    if (lane == 0) atomicSub(&s_task.walking, 1u);
    for (uint32_t spin = 0; spin < (kCoopSpinLimit << 3) && !ring.failed; ++spin) {
      unsigned int left = 0;
      if (lane == 0) left = ld_volatile(&s_task.walking);
      if (__shfl_sync(0xFFFFFFFFu, left, 0) == 0u) break;
      if (!coop_help<APP, CLEAN>(a, &s_task, lane, ring, ring_ptr, &s_flags[warp][0])) ring.failed = true;
      __nanosleep(256);
    }
  }
  if (ring.failed) {
    // A staged copy did not land in time.  Report it, then give the copies this
    // warp may still have in flight one more bounded wait before its shared
    // memory is released with the CTA.
    status |= FW_STATUS_WAIT_TIMEOUT;
#pragma unroll
    for (int t = 0; t < kStages; ++t) mbar_wait(ring.bar + 8u * t, (ring.parity >> t) & 1u);
  }
  // the slots' counters live in lanes 0 .. slots - 1
#pragma unroll
  for (int off = 1; off < slots_of<APP>(); off <<= 1) {
    my_steps += __shfl_xor_sync(0xFFFFFFFFu, my_steps, off);
    my_scanned += __shfl_xor_sync(0xFFFFFFFFu, my_scanned, off);
  }
  status = __reduce_or_sync(0xFFFFFFFFu, status);
  if (lane == 0) {
    if (my_steps) atomicAdd(a.scratch + kSlotSteps, my_steps);
    if (my_scanned) atomicAdd(a.scratch + kSlotScanned, my_scanned);
    if (status) atomicOr(a.scratch + kSlotStatus, (unsigned long long)status);
  }
  if (a.hist_in_smem) {
    __syncthreads();
    for (int z = threadIdx.x; z <= a.d; z += blockDim.x)
      if (s_hist[z]) atomicAdd(a.scratch + kSlotHist + z, (unsigned long long)s_hist[z]);
  }
}

// ---- hub launches: one sweep of a hub's row serves up to 32 walkers ----
//
// Most of what a walk reads are the rows of a few thousand hub vertices, and at any moment many
// walkers sit on the same hub.  The strip totals W(s,l) of a row do not depend on the walker
// (DeepWalk, PPR), only the random words do, so walkers that wait at the same hub are served
// together: the row is swept once by a warp, and after every three supergroups lane q, which
// stands for walker q of the batch, forms walker q's keys for the 96 strips just summed from its
// own Philox blocks (the totals travel by shuffle).  What a walker costs on a hub row drops from
// the row's bytes to one Philox block per three strips, and the bytes are read once per batch.
// The walks are the same as without batching: key, strip id and pick word of every walker are
// what its own sweep would have formed, and the smallest (key, id) wins either way.
//
// A walk call becomes a series of launches on one stream: the walk kernel runs every walker until
// it arrives at a hub and parks it there (hub_park); hub_plan_kernel and hub_scatter_kernel
// group the parked walkers by hub into batches of up to 32; hub_kernel serves the batches and
// parks the walkers whose next vertex is a hub again, lists the others for the walk kernel; and
// so on until nobody is parked.

// Exact test of one strip for one walker, behind the same lower-bound filter as offer_filtered;
// ties go to the lower strip id (the strips of a walker do not arrive in id order here).
__device__ __forceinline__ void offer_lex(Best& b, uint32_t x, uint32_t pick_word, float W, uint32_t id) {
  if (!(W > 0.0f)) return;
  const int g = __clz((int)x);
  const float lower = g ? (float)g : __fmul_rn((float)(x << 1), 0.72f * 0x1p-32f);
  if (lower > __fmul_rn(__fmul_rn(__uint_as_float(b.key), W), 1.000001f)) return;  // NaN bound (nothing yet): passes
  const uint32_t bits = __float_as_uint(__fdiv_rn(fw::exp_key(x), W));
  if (bits < b.key || (bits == b.key && id < b.id)) { b.key = bits; b.id = id; b.pick = pick_word; b.W = W; }
}

// pick_in_row by one lane for its own walker: the strip's quads one after the other from global
// memory (the row was just swept: they come from L2).
template <int APP, bool CLEAN>
__device__ __forceinline__ uint32_t pick_lane(const StepCtx& c, uint32_t B, uint32_t pick, float W) {
  const uint32_t sB = B >> 5, lB = B & 31u;
  const float thr = __fmul_rn((float)(pick >> 8) * 0x1p-24f, W);
  const uint32_t last_blk = (c.nq - 1u) >> 5;
  const uint32_t blk0 = 16u * sB;
  const uint32_t nblk = min(16u, last_blk - blk0 + 1u);
  float acc = 0.0f;
  uint32_t cnt = 0, j = 0, last_pos = 0;
#pragma unroll 1
  for (; j < nblk; ++j) {
    const uint32_t q = 32u * (blk0 + j) + lB;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (q < c.nq) {
      v = plain_bias<APP, CLEAN>(__ldg(c.prim + q), c.want);
      mask_quad(v, q, c.head, c.tail);
    }
    if (v.x > 0.0f) last_pos = 4u * j;
    if (v.y > 0.0f) last_pos = 4u * j + 1u;
    if (v.z > 0.0f) last_pos = 4u * j + 2u;
    if (v.w > 0.0f) last_pos = 4u * j + 3u;
    const float p0 = __fadd_rn(acc, v.x), p1 = __fadd_rn(p0, v.y), p2 = __fadd_rn(p1, v.z);
    acc = __fadd_rn(p2, v.w);
    if (acc <= thr) { cnt += 4u; continue; }
    cnt += (p0 <= thr ? 1u : 0u) + (p1 <= thr ? 1u : 0u) + (p2 <= thr ? 1u : 0u);
    break;
  }
  if (j == nblk) cnt = last_pos;  // rounding pushed u * W past the sequential total: the last positive edge
  return 4u * (32u * (blk0 + (cnt >> 2)) + lB) + (cnt & 3u);
}

// Total bias of strip B by one lane, in the canonical order of the sweep (the same bits).
template <int APP, bool CLEAN>
__device__ __forceinline__ float strip_total_lane(const StepCtx& c, uint32_t B) {
  const uint32_t sB = B >> 5, lB = B & 31u;
  float A[4];
#pragma unroll 1
  for (uint32_t i = 0; i < 4u; ++i) {
    float S[4];
#pragma unroll
    for (uint32_t j = 0; j < 4u; ++j) {
      const uint32_t q = sB * fw::kQuadsPerSuper + i * fw::kQuadsPerSub + 32u * j + lB;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (q < c.nq) {
        v = plain_bias<APP, CLEAN>(__ldg(c.prim + q), c.want);
        mask_quad(v, q, c.head, c.tail);
      }
      S[j] = sum4(v);
    }
    A[i] = sum_strip(S);
  }
  return __fadd_rn(__fadd_rn(A[0], A[1]), __fadd_rn(A[2], A[3]));
}

// Supergroups per part of a split row (a multiple of three: a Philox block serves three).
__host__ __device__ constexpr uint32_t hub_part_supers(uint32_t supers, uint32_t parts) {
  return ((supers + parts - 1u) / parts + 2u) / 3u * 3u;
}

template <int APP, bool CLEAN, typename OffT>
__global__ void __launch_bounds__(kThreads, FW_MIN_BLOCKS) hub_kernel(const __grid_constant__ WalkArgs a) {
  static_assert(APP != FW_APP_NODE2VEC, "strip totals must not depend on the walker (MetaPath: batches are per wanted label)");
  extern __shared__ __align__(128) unsigned char s_dyn[];
  __shared__ __align__(8) unsigned long long s_bar[kWarpsPerCta][2];
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  constexpr uint32_t kRingPerWarp = ring_bytes<APP>();
  uint32_t* s_hist = reinterpret_cast<uint32_t*>(s_dyn + kRingPerWarp * kWarpsPerCta);
  const unsigned char* ring_ptr = s_dyn + kRingPerWarp * warp;
  Ring ring;
  ring.data = smem_addr(ring_ptr);
  ring.bar = smem_addr(&s_bar[warp][0]);
  ring.parity = 0u;
  ring.failed = false;
  if (lane == 0) {
    mbar_init(ring.bar, 1u);
    mbar_init(ring.bar + 8u, 1u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (a.hist_in_smem)
    for (int z = threadIdx.x; z <= a.d; z += blockDim.x) s_hist[z] = 0u;
  __syncthreads();

  const OffT* __restrict__ xadj = static_cast<const OffT*>(a.xadj);
  const int64_t D = (int64_t)a.d + 1;
  const int4* const prim_base = reinterpret_cast<const int4*>(APP == FW_APP_METAPATH ? (const void*)a.label : (const void*)a.weight);
  const int4* const lane_ptr = reinterpret_cast<const int4*>(ring_ptr) + lane;
  const uint32_t n_items = *a.hub.items_n;
  unsigned long long my_steps = 0, my_scanned = 0;
  uint32_t status = 0;

  while (!ring.failed) {
    unsigned long long item = 0;
    if (lane == 0) item = atomicAdd(a.hub.work, 1ull);
    item = __shfl_sync(0xFFFFFFFFu, item, 0);
    if (item >= (unsigned long long)n_items) break;
    const int4 it = __ldg(a.hub.items + item);  // hub index, first entry, entries | part << 8 | parts << 16, group
    const uint32_t n_in = (uint32_t)it.z & 0xFFu, part = ((uint32_t)it.z >> 8) & 0xFFu, parts = (uint32_t)it.z >> 16;
    const int32_t v = __ldg(a.hub.hub_ids + it.x / a.hub.classes);
    const int64_t b = (int64_t)__ldg(xadj + v);
    const uint32_t len = (uint32_t)((int64_t)__ldg(xadj + v + 1) - b);
    const int64_t q0 = b >> 2;
    StepCtx c;
    c.prim = prim_base + q0;
    c.sec = nullptr;
    c.head = (uint32_t)(b - 4 * q0);
    c.tail = c.head + len;
    c.nq = (c.tail + 3u) >> 2;
    c.prev = -1; c.prow = a.adj; c.plen = 0u; c.from = 0u; c.flags = nullptr;
    c.want = APP == FW_APP_METAPATH ? a.schema[it.x % a.hub.classes] : 0;  // the label every walker of the batch wants
    // the walker this lane stands for
    const bool have = lane < n_in;
    const long long qi = have ? (long long)__ldg(a.hub.bucket + it.y + lane) : 0;
    int32_t k = have ? a.hub.kstate[qi] : 0;
    const uint64_t qid = a.qid_base + (uint64_t)qi * a.qid_stride;
    const uint32_t qlo = (uint32_t)qid, qhi = (uint32_t)(qid >> 32);
    const uint32_t c1 = (uint32_t)k | (fw::kPurposeScan << 28);
    Best best{0xFFFFFFFFu, 0xFFFFFFFFu, 0u, 0.0f};

    // ---- one sweep of the row (of this item's part of it); the walkers' keys after every third supergroup ----
    const uint32_t n_half = (c.nq + kHalfQuads - 1u) / kHalfQuads;
    const uint32_t end_super = ((n_half + 1u) >> 1) - 1u;
    // a very long row is split into parts of whole Philox blocks (three supergroups each), one item per part
    const uint32_t per = hub_part_supers(end_super + 1u, parts);
    const uint32_t s_lo = part * per, s_last = min(end_super, s_lo + per - 1u);
    const uint32_t h_end = min(n_half, 2u * (s_last + 1u));
    const bool any = s_lo <= end_super;  // rounding can leave the last parts of a row empty
    if (any && lane == 0) {
      half_fill(c, ring, 2u * s_lo);
      if (2u * s_lo + 1u < h_end) half_fill(c, ring, 2u * s_lo + 1u);
    }
    float W0 = 0.0f, W1 = 0.0f, W2 = 0.0f;
    uint32_t g = s_lo / 3u, m = 0;
#pragma unroll 1
    for (uint32_t sg = s_lo; any; ++sg) {
      const bool last = sg == s_last;
      float W;
      bool ok;
      if (sg == 0u || sg == end_super) ok = super_turn<APP, CLEAN, true>(c, sg, n_half, h_end, lane, ring, lane_ptr, W);
      else ok = super_turn<APP, CLEAN, false>(c, sg, n_half, h_end, lane, ring, lane_ptr, W);
      if (!ok) { ring.failed = true; break; }
      if (m == 0u) W0 = W; else if (m == 1u) W1 = W; else W2 = W;
      if (m == 2u || last) {
        // lane q: walker q's keys for strips (3g .. 3g+2, l), l = 0 .. 31
#pragma unroll 1
        for (int l = 0; l < 32; ++l) {
          const float w0 = __shfl_sync(0xFFFFFFFFu, W0, l), w1 = __shfl_sync(0xFFFFFFFFu, W1, l);
          const float w2 = __shfl_sync(0xFFFFFFFFu, W2, l);
          const fw::Philox4 r = fw::philox4x32_10(g * 32u + (uint32_t)l, c1, qlo, qhi, a.rk);
          offer_lex(best, r.x, r.w, w0, (3u * g) * 32u + (uint32_t)l);
          offer_lex(best, r.y, r.w, w1, (3u * g + 1u) * 32u + (uint32_t)l);
          offer_lex(best, r.z, r.w, w2, (3u * g + 2u) * 32u + (uint32_t)l);
        }
        W0 = 0.0f; W1 = 0.0f; W2 = 0.0f;
        m = 0u;
        ++g;
      } else {
        ++m;
      }
      if (last) break;
    }
    if (ring.failed) break;
    if (parts > 1u) {
      // Split row: every part folds its walkers' best (key, strip id) into the group's words; the
      // part that finds all the others done goes on for the group (nobody waits for anybody).
      if (have && best.id != 0xFFFFFFFFu)
        atomicMin(a.hub.best64 + it.y + lane, ((unsigned long long)best.key << 32) | best.id);
      __threadfence();
      unsigned int before = 0;
      if (lane == 0) before = atomicAdd(a.hub.part_done + it.w, 1u);
      if (__shfl_sync(0xFFFFFFFFu, before, 0) != parts - 1u) continue;
      __threadfence();
      const unsigned long long w = have ? atomicMin(a.hub.best64 + it.y + lane, ~0ull) : ~0ull;  // a coherent read
      best.key = (uint32_t)(w >> 32);
      best.id = (uint32_t)w;
      if (have && best.id != 0xFFFFFFFFu) {  // pick word and total of the winning strip, formed again
        best.pick = fw::philox4x32_10(((best.id >> 5) / 3u) * 32u + (best.id & 31u), c1, qlo, qhi, a.rk).w;
        best.W = strip_total_lane<APP, CLEAN>(c, best.id);
      }
    }

    // ---- every walker takes its step ----
    bool fin = false;
    if (have) {
      if (best.id == 0xFFFFFFFFu) {
        fin = true;  // no edge with a positive bias
      } else {
        const uint32_t rel = pick_lane<APP, CLEAN>(c, best.id, best.pick, best.W);
        const int32_t nxt = __ldg(a.adj + (4 * q0 + (int64_t)rel));
        if (nxt < 0 || (int64_t)nxt >= a.V) {
          status |= FW_STATUS_BAD_NEIGHBOR;
          fin = true;
        } else {
          a.result[qi * D + k + 1] = nxt;
          my_scanned += (unsigned long long)len;
          ++k;
          bool stop = k >= a.d;
          if (APP == FW_APP_PPR) {
            const fw::Philox4 r = fw::philox4x32_10(0u, (uint32_t)(k - 1) | (fw::kPurposeStop << 28), qlo, qhi, a.rk);
            stop = stop || r.x < a.tp_thresh;
          }
          if (stop) {
            fin = true;
          } else {
            // where the walker goes on: parked at the next hub, or listed for the walk kernel
            const OffT nb = __ldg(xadj + nxt), ne = __ldg(xadj + nxt + 1);
            if (ne <= nb) {
              fin = true;  // dead end
            } else if ((uint64_t)(ne - nb) >= (uint64_t)a.hub.min_degree) {
              hub_park(a.hub, qi, k, nxt);
            } else {
              const uint32_t pos = claim_slot(a.hub.next_n);
              a.hub.next_list[pos] = (int32_t)qi;
              a.hub.kstate[qi] = k;
            }
          }
        }
      }
    }
    // ---- close the walks that ended ----
    for (uint32_t mm = __ballot_sync(0xFFFFFFFFu, fin); mm != 0u; mm &= mm - 1u) {
      const int s = __ffs((int)mm) - 1;
      const long long qs = __shfl_sync(0xFFFFFFFFu, qi, s);
      const int ks = __shfl_sync(0xFFFFFFFFu, k, s);
      int32_t* __restrict__ row_out = a.result + qs * D;
      for (int z = ks + 1 + (int)lane; z <= a.d; z += 32) row_out[z] = -1;
    }
    if (fin) {
      my_steps += (unsigned long long)k;
      if (a.hist_in_smem) atomicAdd(&s_hist[k], 1u);
      else atomicAdd(a.scratch + kSlotHist + k, 1ull);
      if (a.hub.fin) a.hub.fin[qi] = a.hub.fin_tag;
    }
  }
  if (ring.failed) {
    status |= FW_STATUS_WAIT_TIMEOUT;
    mbar_wait(ring.bar, ring.parity & 1u);
    mbar_wait(ring.bar + 8u, (ring.parity >> 1) & 1u);
  }
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    my_steps += __shfl_xor_sync(0xFFFFFFFFu, my_steps, off);
    my_scanned += __shfl_xor_sync(0xFFFFFFFFu, my_scanned, off);
  }
  status = __reduce_or_sync(0xFFFFFFFFu, status);
  if (lane == 0) {
    if (my_steps) atomicAdd(a.scratch + kSlotSteps, my_steps);
    if (my_scanned) atomicAdd(a.scratch + kSlotScanned, my_scanned);
    if (status) atomicOr(a.scratch + kSlotStatus, (unsigned long long)status);
  }
  if (a.hist_in_smem) {
    __syncthreads();
    for (int z = threadIdx.x; z <= a.d; z += blockDim.x)
      if (s_hist[z]) atomicAdd(a.scratch + kSlotHist + z, (unsigned long long)s_hist[z]);
  }
}

// The hub kernel of node2vec.  The sweep of a row reads plain weights, which do not depend on the
// walker; what does -- the bias factors 1/p, 1, 1/q by the walker's previous vertex -- enters per
// strip, and only for the strips whose optimistic key can still win (n2v_test).  So the row is swept
// once per batch, and after every third supergroup the warp goes through the batch walker by walker:
// the lanes stand for the strips, as in a walker's own sweep, and form that walker's Philox words;
// n2v_test evaluates the few strips it has to.  A walker's best (key, strip, pick word, total) lives
// in the registers of the lane with the walker's number between its turns.  Rows are not split.
template <bool CLEAN, typename OffT>
__global__ void __launch_bounds__(kThreads, FW_MIN_BLOCKS) hub_kernel_n2v(const __grid_constant__ WalkArgs a) {
  constexpr int SAPP = kAppPlainCompact;  // plain weights
  extern __shared__ __align__(128) unsigned char s_dyn[];
  __shared__ __align__(8) unsigned long long s_bar[kWarpsPerCta][2];
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  constexpr uint32_t kRingPerWarp = ring_bytes<FW_APP_DEEPWALK>();
  uint32_t* s_hist = reinterpret_cast<uint32_t*>(s_dyn + kRingPerWarp * kWarpsPerCta);
  const unsigned char* ring_ptr = s_dyn + kRingPerWarp * warp;
  Ring ring;
  ring.data = smem_addr(ring_ptr);
  ring.bar = smem_addr(&s_bar[warp][0]);
  ring.parity = 0u;
  ring.failed = false;
  if (lane == 0) {
    mbar_init(ring.bar, 1u);
    mbar_init(ring.bar + 8u, 1u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (a.hist_in_smem)
    for (int z = threadIdx.x; z <= a.d; z += blockDim.x) s_hist[z] = 0u;
  __syncthreads();

  const OffT* __restrict__ xadj = static_cast<const OffT*>(a.xadj);
  const int64_t D = (int64_t)a.d + 1;
  const int4* const prim_base = reinterpret_cast<const int4*>(a.weight);
  const int4* const sec_base = reinterpret_cast<const int4*>(a.adj);
  const int4* const lane_ptr = reinterpret_cast<const int4*>(ring_ptr) + lane;
  const uint32_t n_items = *a.hub.items_n;
  unsigned long long my_steps = 0, my_scanned = 0;
  uint32_t status = 0;

  while (!ring.failed) {
    unsigned long long item = 0;
    if (lane == 0) item = atomicAdd(a.hub.work, 1ull);
    item = __shfl_sync(0xFFFFFFFFu, item, 0);
    if (item >= (unsigned long long)n_items) break;
    const int4 it = __ldg(a.hub.items + item);
    const uint32_t n_in = (uint32_t)it.z & 0xFFu;
    const int32_t v = __ldg(a.hub.hub_ids + it.x);
    const int64_t b = (int64_t)__ldg(xadj + v);
    const uint32_t len = (uint32_t)((int64_t)__ldg(xadj + v + 1) - b);
    const int64_t q0 = b >> 2;
    StepCtx c;
    c.prim = prim_base + q0;
    c.sec = sec_base + q0;
    c.head = (uint32_t)(b - 4 * q0);
    c.tail = c.head + len;
    c.nq = (c.tail + 3u) >> 2;
    c.prev = -1; c.prow = a.adj; c.plen = 0u; c.want = 0; c.from = 0u; c.flags = nullptr;
    // the walker of this lane: query, steps so far, previous vertex and its row
    const bool have = lane < n_in;
    const long long qi = have ? (long long)__ldg(a.hub.bucket + it.y + lane) : 0;
    int32_t k = have ? a.hub.kstate[qi] : 0;
    const uint64_t qid = a.qid_base + (uint64_t)qi * a.qid_stride;
    const uint32_t qlo = (uint32_t)qid, qhi = (uint32_t)(qid >> 32);
    int32_t wprev = -1;
    long long wpb = 0;
    uint32_t wplen = 0;
    if (have && k > 0) {
      wprev = a.result[qi * D + k - 1];
      wpb = (long long)__ldg(xadj + wprev);
      wplen = (uint32_t)((long long)__ldg(xadj + wprev + 1) - wpb);
    }
    uint32_t bkey = 0xFFFFFFFFu, bid = 0xFFFFFFFFu, bpick = 0u;
    float bW = 0.0f;

    const uint32_t n_half = (c.nq + kHalfQuads - 1u) / kHalfQuads;
    const uint32_t end_super = ((n_half + 1u) >> 1) - 1u;
    if (lane == 0) {
      half_fill(c, ring, 0u);
      if (n_half > 1u) half_fill(c, ring, 1u);
    }
    float W0 = 0.0f, W1 = 0.0f, W2 = 0.0f;
    uint32_t g = 0, m = 0;
#pragma unroll 1
    for (uint32_t sg = 0;; ++sg) {
      const bool last = sg == end_super;
      float W;
      bool ok;
      if (sg == 0u || last) ok = super_turn<SAPP, CLEAN, true>(c, sg, n_half, n_half, lane, ring, lane_ptr, W);
      else ok = super_turn<SAPP, CLEAN, false>(c, sg, n_half, n_half, lane, ring, lane_ptr, W);
      if (!ok) { ring.failed = true; break; }
      if (m == 0u) W0 = W; else if (m == 1u) W1 = W; else W2 = W;
      if (m == 2u || last) {
        // the batch, walker by walker: lanes are strips
#pragma unroll 1
        for (uint32_t q = 0; q < n_in; ++q) {
          c.prev = __shfl_sync(0xFFFFFFFFu, wprev, (int)q);
          c.prow = a.adj + __shfl_sync(0xFFFFFFFFu, wpb, (int)q);
          c.plen = __shfl_sync(0xFFFFFFFFu, wplen, (int)q);
          const uint32_t c1 = (uint32_t)__shfl_sync(0xFFFFFFFFu, k, (int)q) | (fw::kPurposeScan << 28);
          const uint32_t ql = __shfl_sync(0xFFFFFFFFu, qlo, (int)q), qh = __shfl_sync(0xFFFFFFFFu, qhi, (int)q);
          Best best{__shfl_sync(0xFFFFFFFFu, bkey, (int)q), __shfl_sync(0xFFFFFFFFu, bid, (int)q),
                    __shfl_sync(0xFFFFFFFFu, bpick, (int)q), __shfl_sync(0xFFFFFFFFu, bW, (int)q)};
          const fw::Philox4 r = fw::philox4x32_10(g * 32u + lane, c1, ql, qh, a.k0, a.k1);
#pragma unroll 1
          for (uint32_t i = 0; i <= m; ++i) {
            const float Wi = i == 0u ? W0 : i == 1u ? W1 : W2;
            const uint32_t x = i == 0u ? r.x : i == 1u ? r.y : r.z;
            const uint32_t s = 3u * g + i;
            if (c.prev >= 0) {
              n2v_test<CLEAN>(a, c, s, lane, Wi, x, r.w, best);
            } else {
              // first step of a query that starts at the hub: plain weights, every strip's key
              uint32_t key = 0xFFFFFFFFu, id = 0xFFFFFFFFu;
              if (Wi > 0.0f) { key = __float_as_uint(__fdiv_rn(fw::exp_key(x), Wi)); id = s * 32u + lane; }
              warp_argmin(key, id);
              if (id != 0xFFFFFFFFu && (key < best.key || (key == best.key && id < best.id))) {
                best.key = key; best.id = id;
                best.pick = __shfl_sync(0xFFFFFFFFu, r.w, (int)(id & 31u));
                best.W = __shfl_sync(0xFFFFFFFFu, Wi, (int)(id & 31u));
              }
            }
          }
          if (lane == q) { bkey = best.key; bid = best.id; bpick = best.pick; bW = best.W; }
        }
        W0 = 0.0f; W1 = 0.0f; W2 = 0.0f;
        m = 0u;
        ++g;
      } else {
        ++m;
      }
      if (last) break;
    }
    if (ring.failed) break;

    // ---- the pick inside every walker's winning strip, walker by walker ----
    uint32_t rel = 0xFFFFFFFFu;
#pragma unroll 1
    for (uint32_t q = 0; q < n_in; ++q) {
      const uint32_t B = __shfl_sync(0xFFFFFFFFu, bid, (int)q);
      if (B == 0xFFFFFFFFu) continue;  // warp-uniform
      c.prev = __shfl_sync(0xFFFFFFFFu, wprev, (int)q);
      c.prow = a.adj + __shfl_sync(0xFFFFFFFFu, wpb, (int)q);
      c.plen = __shfl_sync(0xFFFFFFFFu, wplen, (int)q);
      const uint32_t pick = __shfl_sync(0xFFFFFFFFu, bpick, (int)q);
      const float WB = __shfl_sync(0xFFFFFFFFu, bW, (int)q);
      const uint32_t r1 = c.prev >= 0 ? n2v_pick<CLEAN>(a, c, B, pick, lane) : pick_in_row<SAPP, CLEAN>(a, c, B, pick, WB, lane);
      if (lane == q) rel = r1;
    }

    // ---- every walker takes its step ----
    bool fin = false;
    if (have) {
      if (rel == 0xFFFFFFFFu) {
        fin = true;  // no edge with a positive bias
      } else {
        const int32_t nxt = __ldg(a.adj + (4 * q0 + (int64_t)rel));
        if (nxt < 0 || (int64_t)nxt >= a.V) {
          status |= FW_STATUS_BAD_NEIGHBOR;
          fin = true;
        } else {
          a.result[qi * D + k + 1] = nxt;
          my_scanned += (unsigned long long)len;
          ++k;
          if (k >= a.d) {
            fin = true;
          } else {
            const OffT nb = __ldg(xadj + nxt), ne = __ldg(xadj + nxt + 1);
            if (ne <= nb) {
              fin = true;  // dead end
            } else if ((uint64_t)(ne - nb) >= (uint64_t)a.hub.min_degree) {
              hub_park(a.hub, qi, k, nxt);
            } else {
              const uint32_t pos = claim_slot(a.hub.next_n);
              a.hub.next_list[pos] = (int32_t)qi;
              a.hub.kstate[qi] = k;
            }
          }
        }
      }
    }
    for (uint32_t mm = __ballot_sync(0xFFFFFFFFu, fin); mm != 0u; mm &= mm - 1u) {
      const int s = __ffs((int)mm) - 1;
      const long long qs = __shfl_sync(0xFFFFFFFFu, qi, s);
      const int ks = __shfl_sync(0xFFFFFFFFu, k, s);
      int32_t* __restrict__ row_out = a.result + qs * D;
      for (int z = ks + 1 + (int)lane; z <= a.d; z += 32) row_out[z] = -1;
    }
    if (fin) {
      my_steps += (unsigned long long)k;
      if (a.hist_in_smem) atomicAdd(&s_hist[k], 1u);
      else atomicAdd(a.scratch + kSlotHist + k, 1ull);
      if (a.hub.fin) a.hub.fin[qi] = a.hub.fin_tag;
    }
  }
  if (ring.failed) {
    status |= FW_STATUS_WAIT_TIMEOUT;
    mbar_wait(ring.bar, ring.parity & 1u);
    mbar_wait(ring.bar + 8u, (ring.parity >> 1) & 1u);
  }
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    my_steps += __shfl_xor_sync(0xFFFFFFFFu, my_steps, off);
    my_scanned += __shfl_xor_sync(0xFFFFFFFFu, my_scanned, off);
  }
  status = __reduce_or_sync(0xFFFFFFFFu, status);
  if (lane == 0) {
    if (my_steps) atomicAdd(a.scratch + kSlotSteps, my_steps);
    if (my_scanned) atomicAdd(a.scratch + kSlotScanned, my_scanned);
    if (status) atomicOr(a.scratch + kSlotStatus, (unsigned long long)status);
  }
  if (a.hist_in_smem) {
    __syncthreads();
    for (int z = threadIdx.x; z <= a.d; z += blockDim.x)
      if (s_hist[z]) atomicAdd(a.scratch + kSlotHist + z, (unsigned long long)s_hist[z]);
  }
}

// Groups the parked walkers by hub (a key is a hub and class).  Two launches over tiles of
// kPlanTile keys: hub_plan_count adds up every tile's walkers and batch items, and the CTA that
// finishes last turns the tile totals into offsets; hub_plan_emit then writes every key's first
// bucket entry (`base`), one item per 32 walkers of a key and part of the hub's row, and sets the
// counts and the scatter cursors back to zero.
constexpr int kPlanThreads = 1024, kPlanKeys = 4, kPlanTile = kPlanThreads * kPlanKeys;
constexpr int kPlanMaxTiles = 1 << 16;

// Sums (walkers, items) of the thread's kPlanKeys keys; exclusive offsets of the thread within the
// CTA in (xc, xb), the CTA's totals in s_tot.  All threads of the CTA call it.
__device__ __forceinline__ void plan_tile_scan(uint32_t my_c, uint32_t my_b, uint32_t& xc, uint32_t& xb, uint32_t* s_wc,
                                               uint32_t* s_wb, uint32_t* s_tot) {
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  uint32_t ic = my_c, ib = my_b;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t x = __shfl_up_sync(0xFFFFFFFFu, ic, off), y = __shfl_up_sync(0xFFFFFFFFu, ib, off);
    if (lane >= off) { ic += x; ib += y; }
  }
  if (lane == 31) { s_wc[warp] = ic; s_wb[warp] = ib; }
  __syncthreads();
  if (warp == 0) {
    const uint32_t wc = s_wc[lane], wb = s_wb[lane];
    uint32_t c = wc, b = wb;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t x = __shfl_up_sync(0xFFFFFFFFu, c, off), y = __shfl_up_sync(0xFFFFFFFFu, b, off);
      if (lane >= off) { c += x; b += y; }
    }
    s_wc[lane] = c - wc;
    s_wb[lane] = b - wb;
    if (lane == 31) { s_tot[0] = c; s_tot[1] = b; }
  }
  __syncthreads();
  xc = s_wc[warp] + ic - my_c;
  xb = s_wb[warp] + ib - my_b;
}

__global__ void __launch_bounds__(kPlanThreads) hub_plan_count(const uint32_t* __restrict__ cnt, const uint16_t* __restrict__ parts,
                                                               int n_keys, int classes, uint2* tile_tot, uint32_t* tiles_done,
                                                               uint32_t* items_n) {
  __shared__ uint32_t s_wc[32], s_wb[32], s_tot[2];
  __shared__ bool s_last;
  const int t = threadIdx.x, k0 = blockIdx.x * kPlanTile + t * kPlanKeys;
  uint32_t my_c = 0, my_b = 0;
#pragma unroll
  for (int i = 0; i < kPlanKeys; ++i)
    if (k0 + i < n_keys) {
      const uint32_t n = cnt[k0 + i];
      my_c += n;
      my_b += ((n + 31u) >> 5) * parts[(k0 + i) / classes];
    }
  uint32_t xc, xb;
  plan_tile_scan(my_c, my_b, xc, xb, s_wc, s_wb, s_tot);
  if (t == 0) {
    tile_tot[blockIdx.x] = make_uint2(s_tot[0], s_tot[1]);
    __threadfence();
    s_last = atomicAdd(tiles_done, 1u) == gridDim.x - 1u;
  }
  __syncthreads();
  if (!s_last) return;
  // the last CTA: tile totals -> exclusive tile offsets, in place (nobody waits for anybody)
  __threadfence();
  uint32_t carry_c = 0, carry_b = 0;
  for (int base = 0; base < (int)gridDim.x; base += kPlanThreads) {
    const int i = base + t;
    uint2 v = make_uint2(0u, 0u);
    if (i < (int)gridDim.x) v = __ldcg(tile_tot + i);  // written by other CTAs: read at L2
    __syncthreads();  // s_tot of the round before has been read
    plan_tile_scan(v.x, v.y, xc, xb, s_wc, s_wb, s_tot);
    if (i < (int)gridDim.x) tile_tot[i] = make_uint2(carry_c + xc, carry_b + xb);
    carry_c += s_tot[0];
    carry_b += s_tot[1];
  }
  if (t == 0) {
    *items_n = carry_b;
    *tiles_done = 0u;
  }
}

__global__ void __launch_bounds__(kPlanThreads) hub_plan_emit(uint32_t* cnt, uint32_t* base, uint32_t* fill, int4* items,
                                                              const uint16_t* __restrict__ parts, uint32_t* part_done, int n_keys,
                                                              int classes, const uint2* __restrict__ tile_off) {
  __shared__ uint32_t s_wc[32], s_wb[32], s_tot[2];
  // keys with many batches: their items are written by a warp each, its lanes side by side (one
  // thread would take as long as the rest of the round's planning together for the busiest hubs)
  // (and the few keys with thousands of batches by the whole CTA)
  constexpr uint32_t kBigGroups = 64, kBigCap = 1024, kHugeGroups = 2048, kHugeCap = 32;
  __shared__ uint32_t s_big_n, s_big[kBigCap][5], s_huge_n, s_huge[kHugeCap][5];
  const int t = threadIdx.x, k0 = blockIdx.x * kPlanTile + t * kPlanKeys;
  if (t == 0) { s_big_n = 0u; s_huge_n = 0u; }
  uint32_t n[kPlanKeys], np[kPlanKeys], my_c = 0, my_b = 0;
#pragma unroll
  for (int i = 0; i < kPlanKeys; ++i) {
    n[i] = 0u;
    np[i] = 0u;
    if (k0 + i < n_keys) {
      n[i] = cnt[k0 + i];
      np[i] = parts[(k0 + i) / classes];
      my_c += n[i];
      my_b += ((n[i] + 31u) >> 5) * np[i];
    }
  }
  uint32_t xc, xb;
  plan_tile_scan(my_c, my_b, xc, xb, s_wc, s_wb, s_tot);
  const uint2 off0 = tile_off[blockIdx.x];
  uint32_t at = off0.x + xc, it = off0.y + xb;
#pragma unroll
  for (int i = 0; i < kPlanKeys; ++i)
    if (k0 + i < n_keys) {
      base[k0 + i] = at;
      const uint32_t groups = (n[i] + 31u) >> 5;
      uint32_t slot = kBigCap, hslot = kHugeCap;
      if (groups > kHugeGroups) hslot = atomicAdd(&s_huge_n, 1u);
      if (hslot >= kHugeCap && groups > kBigGroups) slot = atomicAdd(&s_big_n, 1u);
      if (hslot < kHugeCap) {
        s_huge[hslot][0] = (uint32_t)(k0 + i); s_huge[hslot][1] = n[i]; s_huge[hslot][2] = np[i]; s_huge[hslot][3] = at; s_huge[hslot][4] = it;
        it += groups * np[i];
      } else if (slot < kBigCap) {
        s_big[slot][0] = (uint32_t)(k0 + i); s_big[slot][1] = n[i]; s_big[slot][2] = np[i]; s_big[slot][3] = at; s_big[slot][4] = it;
        it += groups * np[i];
      } else {
        for (uint32_t off = 0; off < n[i]; off += 32u) {
          const uint32_t group = it;
          part_done[group] = 0u;
          for (uint32_t p = 0; p < np[i]; ++p)
            items[it++] = make_int4(k0 + i, (int)(at + off), (int)(min(32u, n[i] - off) | (p << 8) | (np[i] << 16)), (int)group);
        }
      }
      at += n[i];
      if (n[i] != 0u) cnt[k0 + i] = 0u;
      fill[k0 + i] = 0u;
    }
  __syncthreads();
  const uint32_t huge = min(s_huge_n, kHugeCap);
  for (uint32_t e = 0; e < huge; ++e) {
    const uint32_t key = s_huge[e][0], kn = s_huge[e][1], knp = s_huge[e][2], kat = s_huge[e][3], kit = s_huge[e][4];
    const uint32_t work = ((kn + 31u) >> 5) * knp;  // one item per thread and turn
    for (uint32_t w = (uint32_t)t; w < work; w += kPlanThreads) {
      const uint32_t j = w / knp, p = w - j * knp, group = kit + j * knp, off = 32u * j;
      if (p == 0u) part_done[group] = 0u;
      items[group + p] = make_int4((int)key, (int)(kat + off), (int)(min(32u, kn - off) | (p << 8) | (knp << 16)), (int)group);
    }
  }
  const uint32_t big = min(s_big_n, kBigCap);
  for (uint32_t e = (uint32_t)t >> 5; e < big; e += kPlanThreads / 32) {
    const uint32_t key = s_big[e][0], kn = s_big[e][1], knp = s_big[e][2], kat = s_big[e][3], kit = s_big[e][4];
    for (uint32_t j = (uint32_t)t & 31u; j < (kn + 31u) >> 5; j += 32u) {
      const uint32_t group = kit + j * knp, off = 32u * j;
      part_done[group] = 0u;
      for (uint32_t p = 0; p < knp; ++p)
        items[group + p] = make_int4((int)key, (int)(kat + off), (int)(min(32u, kn - off) | (p << 8) | (knp << 16)), (int)group);
    }
  }
}

__global__ void hub_scatter_kernel(const int32_t* __restrict__ park_hub, const int32_t* __restrict__ park_qi,
                                   const uint32_t* __restrict__ park_n, const uint32_t* __restrict__ base, uint32_t* fill,
                                   int32_t* __restrict__ bucket) {
  const uint32_t n = *park_n;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int32_t h = park_hub[i];
    bucket[base[h] + atomicAdd(fill + h, 1u)] = park_qi[i];
  }
}

// Early delivery of a hub-batched call's result.  The caller's walk table is page-locked host memory
// the device can write (`host`, same layout as `result`).  Every walk that ends leaves the tag of its
// launch in fin[query]; after each round of the series this kernel runs on a stream of its own and
// copies the rows whose tag lies in (lo, hi] -- all of them written by launches that are complete --
// to the host table while the next rounds walk on, so that the table's trip over PCIe (as long as
// half a pass for 80-step walks) hides behind the walk instead of following it.  Tags above hi (walks
// ending in launches that run beside this kernel) are left to a later launch; the last one takes
// every tag left.  A warp looks at 128 queries at a time and copies four rows side by side, in
// 128-byte segments aligned in the host table.  A few CTAs of 1,024 threads: what limits the kernel
// is the round trip of its stores over PCIe, so it needs many warps in flight, and every SM it sits
// on is one the walk kernels share (measured on config 2, whole call: 4 CTAs 79 ms -- delivery falls
// behind --, 6 CTAs 63 ms, 8 CTAs 64-65 ms, 12 CTAs 67 ms, 32 CTAs of 256 threads 68 ms, one copy
// after the last launch 76.5 ms).
constexpr int kDeliverThreads = 1024;
constexpr int kDeliverRows = 4;  // rows a warp copies side by side
struct DeliverCtl {
  unsigned int rows;  // rows that have been written to the host table by the launches so far
  unsigned int stop;  // set by the host: the table will travel in one copy after all, give up
};
__global__ void __launch_bounds__(kDeliverThreads) deliver_kernel(const int32_t* __restrict__ result, int32_t* __restrict__ host,
                                                                  const int32_t* fin, long long n, int D, int lo, int hi,
                                                                  DeliverCtl* ctl) {
  const uint32_t lane = threadIdx.x & 31u;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int segs = (D + 31 + 31) / 32;  // segments of 32 cells a row can touch
  for (long long base = warp * 128; base < n; base += warps * 128) {
    if (ld_volatile(&ctl->stop) != 0u) return;
    const long long q4 = base + 4 * (long long)lane;
    int f[4] = {0, 0, 0, 0};
    if (q4 + 3 < n) {
      const int4 v = __ldcg(reinterpret_cast<const int4*>(fin + q4));
      f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    } else {
      for (int c = 0; c < 4; ++c) if (q4 + c < n) f[c] = __ldcg(fin + q4 + c);
    }
    // bit 4 l + c of the warp's 128-bit mask: query base + 4 l + c is to be delivered
    uint32_t m[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) m[c] = __ballot_sync(0xFFFFFFFFu, f[c] > lo && f[c] <= hi);
    const unsigned int found = __popc(m[0]) + __popc(m[1]) + __popc(m[2]) + __popc(m[3]);
    int c = 0;
    while (c < 4) {
      long long o[kDeliverRows];
      int z0[kDeliverRows];
      int rows = 0;
#pragma unroll
      for (int r = 0; r < kDeliverRows; ++r) {
        while (c < 4 && m[c] == 0u) ++c;
        o[r] = -1; z0[r] = 0;
        if (c < 4) {
          const long long q = base + 4 * (long long)(__ffs((int)m[c]) - 1) + c;
          m[c] &= m[c] - 1u;
          o[r] = q * D;
          z0[r] = (int)lane - (int)(((uintptr_t)(host + o[r]) >> 2) & 31u);
          ++rows;
        }
      }
      if (rows == 0) break;
      for (int t = 0; t < segs; ++t) {
        int32_t v[kDeliverRows];
        bool u[kDeliverRows];
#pragma unroll
        for (int r = 0; r < kDeliverRows; ++r) {
          const int z = z0[r] + 32 * t;
          u[r] = o[r] >= 0 && z >= 0 && z < D;
          v[r] = 0;
          if (u[r]) v[r] = __ldcs(result + o[r] + z);
        }
#pragma unroll
        for (int r = 0; r < kDeliverRows; ++r)
          if (u[r]) host[o[r] + z0[r] + 32 * t] = v[r];
      }
    }
    if (found != 0u && lane == 0) atomicAdd(&ctl->rows, found);
  }
}

using KernelFn = void (*)(const WalkArgs);

// The kernels of a hub-batched call: the walk kernel that parks walkers at hubs, and the hub kernel.
template <int APP, int HUBS>
inline KernelFn pick_hub_walk(bool clean, int xadj_bits) {
  if (xadj_bits == 64)
    return clean ? (KernelFn)walk_kernel<APP, FW_GROUP_STRIP, true, int64_t, HUBS> : (KernelFn)walk_kernel<APP, FW_GROUP_STRIP, false, int64_t, HUBS>;
  return clean ? (KernelFn)walk_kernel<APP, FW_GROUP_STRIP, true, uint32_t, HUBS> : (KernelFn)walk_kernel<APP, FW_GROUP_STRIP, false, uint32_t, HUBS>;
}
template <int APP>
inline KernelFn pick_hub_serve(bool clean, int xadj_bits) {
  if (xadj_bits == 64) return clean ? (KernelFn)hub_kernel<APP, true, int64_t> : (KernelFn)hub_kernel<APP, false, int64_t>;
  return clean ? (KernelFn)hub_kernel<APP, true, uint32_t> : (KernelFn)hub_kernel<APP, false, uint32_t>;
}
// which: 0 the walk kernel that parks at hubs of 1,016 neighbours, 3 of 504, 1 the hub kernel,
// 2 the walk kernel of the tail
template <int APP>
inline KernelFn pick_hub_kernel_of(int which, bool clean, int xadj_bits) {
  return which == 1 ? pick_hub_serve<APP>(clean, xadj_bits)
       : which == 2 ? pick_hub_walk<APP, kHubTail>(clean, xadj_bits)
       : which == 3 ? pick_hub_walk<APP, kHubParkLow>(clean, xadj_bits) : pick_hub_walk<APP, kHubPark>(clean, xadj_bits);
}
inline KernelFn pick_hub_kernel_n2v(int which, bool clean, int xadj_bits) {
  if (which == 1) {
    if (xadj_bits == 64) return clean ? (KernelFn)hub_kernel_n2v<true, int64_t> : (KernelFn)hub_kernel_n2v<false, int64_t>;
    return clean ? (KernelFn)hub_kernel_n2v<true, uint32_t> : (KernelFn)hub_kernel_n2v<false, uint32_t>;
  }
  return which == 2 ? pick_hub_walk<FW_APP_NODE2VEC, kHubTail>(clean, xadj_bits) : pick_hub_walk<FW_APP_NODE2VEC, kHubPark>(clean, xadj_bits);
}
inline KernelFn pick_hub_kernel(int app, int which, bool clean, int xadj_bits) {
  if (app == FW_APP_NODE2VEC) return pick_hub_kernel_n2v(which, clean, xadj_bits);
  if (app == FW_APP_PPR) return pick_hub_kernel_of<FW_APP_PPR>(which, clean, xadj_bits);
  if (app == FW_APP_METAPATH) return pick_hub_kernel_of<FW_APP_METAPATH>(which, true, xadj_bits);  // 0/1 biases: nothing to clamp
  return pick_hub_kernel_of<FW_APP_DEEPWALK>(which, clean, xadj_bits);
}

template <int APP, int MODE, bool CLEAN>
inline KernelFn pick_off(int xadj_bits) {
  return xadj_bits == 64 ? (KernelFn)walk_kernel<APP, MODE, CLEAN, int64_t>
                         : (KernelFn)walk_kernel<APP, MODE, CLEAN, uint32_t>;
}
template <int APP>
inline KernelFn pick_mode(int mode, bool clean, bool shared, int xadj_bits) {
  if (mode == FW_GROUP_EDGE) return pick_off<APP, FW_GROUP_EDGE, false>(xadj_bits);
  if (shared)
    return clean ? pick_off<APP, kModeStripShared, true>(xadj_bits) : pick_off<APP, kModeStripShared, false>(xadj_bits);
  return clean ? pick_off<APP, FW_GROUP_STRIP, true>(xadj_bits) : pick_off<APP, FW_GROUP_STRIP, false>(xadj_bits);
}
// clean: all weights are known to be >= 0 and not NaN; shared: warps share very long rows
inline KernelFn pick_kernel(int app, int mode, bool clean, bool shared, int xadj_bits) {
  switch (app) {
    case FW_APP_DEEPWALK: return pick_mode<FW_APP_DEEPWALK>(mode, clean, shared, xadj_bits);
    case FW_APP_PPR: return pick_mode<FW_APP_PPR>(mode, clean, shared, xadj_bits);
    case FW_APP_NODE2VEC: return pick_mode<FW_APP_NODE2VEC>(mode, clean, shared, xadj_bits);
    default:  // MetaPath biases are 0/1: nothing to clamp
      return pick_mode<FW_APP_METAPATH>(mode, true, shared, xadj_bits);
  }
}

// Dynamic shared memory of a CTA of the walk kernel of a hub-batched call.
inline size_t hub_walk_smem_bytes(uint32_t hub_limit, int d, bool hist_in_smem) {
  return (size_t)kWarpsPerCta * 2u * 16u * staged_quads(hub_limit) + (hist_in_smem ? (size_t)(d + 1) * 4 : 0);
}

// Dynamic shared memory of one CTA: the warps' rings, then the histogram.
inline size_t kernel_smem_bytes(int app, int mode, int d, bool hist_in_smem) {
  size_t ring = 0;
  if (mode != FW_GROUP_EDGE)
    ring = (size_t)kWarpsPerCta * (app == FW_APP_NODE2VEC ? ring_bytes<FW_APP_NODE2VEC>() : ring_bytes<FW_APP_DEEPWALK>());
  return ring + (hist_in_smem ? (size_t)(d + 1) * 4 : 0);
}

}  // namespace fwk
