// Random-walk engine for sm_100a: persistent kernel, global atomic query
// counter, exponential-race reservoir sampler, Philox keyed by (query, step).
//
// Stands in for the reference's production scheduler kernels
// (include/walker.cuh:1307-1442 and 1444-1580), its warp/block samplers
// (include/sampler.cuh:46-200), the four walker classes (include/app.cuh:58-152),
// the per-query Task (include/gpu_task.cuh:24-78), the XORWOW stream
// (include/myrand.cuh) and the host launch slice (src/walk.cu:373-466, 527-649).
//
// Sampling law per step: P(edge i) = bias_i / sum(bias), as the reference's
// prefix-sum reservoir gives (include/sampler.cuh:46-85).  Mechanism: each
// candidate group draws key = E / W (E exponential from Philox, W the group's
// total bias); the smallest (key, group id) wins.  min is associative and
// commutative, so the result does not depend on which lane, warp or CTA
// looked at which part of the row, and a CPU walker using the same stream
// reproduces every walk bit for bit.
#include <cuda_runtime.h>

#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <chrono>
#include <functional>
#include <mutex>
#include <new>
#include <vector>

#include "fw_internal.h"
#include "fw_kernels.cuh"
#include "fw_spec.cuh"

using namespace fwk;

// Graphs with a row of at least this many edges run the kernel variant whose warps share very
// long rows (a single warp on a row of 10^6 edges is what the tail of a launch consists of).
static constexpr int64_t kSharingAutoDegree = 262144;

// Hub batching: vertices of at least this many neighbours are hubs (about the reference's limit
// between its warp and its block sampler, 1,024: include/walker.cuh:29).
// A call uses the lower hub limit when it brings at least this many queries per hub of that limit
// (measured on R-MAT scale 22, 19,324 hubs of the lower limit and 9,109 of the higher: 2,097,152
// queries, 108 per hub, 31.4 ms against 32.6 with the higher limit; 1,048,576 queries 21.2 against
// 20.5; scale 24, 10^7 PPR queries, about 50 per hub: 31 ms against 24).
static constexpr int64_t kHubDenseQueries = 100;
// A call is hub-batched at all when it brings at least this many queries per hub of the higher
// limit: every round of the series has a fixed cost (its launches, the longest single sweep, one
// read-back), which a short call does not earn back (R-MAT scale 22: 524,288 queries, 57 per hub,
// take 15.0 ms batched and 15.2 in one launch; 1,048,576, 115 per hub, 20.5 ms against 27.8;
// 2,097,152 31.4 against 53.3; 262,144 12.5 batched).
static constexpr int64_t kHubMinQueries = 64;
static constexpr int64_t kHubMax = (int64_t)1 << 22;
static constexpr int64_t kHubPartSupers = 24;  // supergroups (49,152 neighbours) of a hub's row per sweeping warp, about
static constexpr int64_t kHubMaxParts = 64;
// A call goes to its tail launch when the walkers left parked would, sweeping alone, scan fewer than
// this many neighbours in their next hub step (parked x mean row length of a hub): about what two
// rounds cost in launches and read-backs.  Measured, ms per pass at 2e8 / 4e8-5e8 / 1e9 and with the
// earlier rule of a sixteenth of the queries: config 2 52.0 / 52.1 / 53.1 / 52.0; PPR on the same
// graph 6.07 / 6.09 / 6.35 / 5.93; config 3 20.96 / 20.42 / 21.56 / 25.25; config 5 61.2 / 61.2 / 61.2 / 65.9.
static constexpr double kHubTailEdges = 4e8;
static constexpr int64_t kHubTailMin = 2048;   // ... always once fewer than this many are left, never with a quarter of the queries or more
// CTAs (of 1,024 threads) of a deliver_kernel launch: as few as keep up with the walk (see deliver_kernel).
static constexpr int kDeliverCtas = 8;
static constexpr int kDeliverMinCells = 32;       // shortest result row (d + 1) early delivery takes on
static constexpr double kLinkBytesPerUs = 50e3;   // what a walk table is assumed to need on the host link: 50 GB/s

// Device control words of one round of a hub-batched call.
struct HubCtl {
  unsigned long long work_walk;  // work counter of the round's walk kernel
  unsigned long long work_hub;   // ... of its hub kernel
  uint32_t park_n;               // walkers parked for this round's hub kernel
  uint32_t list_n;               // walkers listed for this round's walk kernel
  uint32_t items_n;              // batches of this round's hub kernel
  uint32_t tiles_done;           // plan: tiles counted (back to zero when the last one is)
};


// ---------------------------------------------------------------------------
// Engine
// ---------------------------------------------------------------------------

struct fw_engine {
  std::mutex mu;  // an engine serves one walk call at a time; calls from several threads queue here
  int device = 0;
  int sms = 0;
  int64_t V = 0, E = 0;
  int xadj_bits = 32;
  bool clean_weights = false;  // every weight is >= 0 and not NaN: the kernels skip the clamp
  int64_t max_degree = 0;
  int sharing = -1;            // warps share very long rows: -1 by max degree, 0 never, 1 always
  void* d_xadj = nullptr;
  int32_t* d_adj = nullptr;
  float* d_weight = nullptr;
  int32_t* d_label = nullptr;
  unsigned long long* d_scratch = nullptr;  // counters + histogram
  unsigned long long* h_scratch = nullptr;  // pinned mirror
  size_t scratch_words = 0;
  cudaStream_t stream = nullptr, stream2 = nullptr;
  cudaEvent_t ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  // early delivery of a hub-batched call's result into page-locked host memory (deliver_kernel)
  int early_delivery = -1;         // -1: where the table is host memory the device can write and the walk is long
                                   // enough, 0: never, 1: from the first launch on, 2: as 1 with the fallback copy
  cudaStream_t stream_out = nullptr;
  cudaEvent_t ev_round = nullptr;  // end of a round's launches on the walk stream
  cudaEvent_t ev_out = nullptr;    // end of the last deliver_kernel launch of a call
  int32_t* d_fin = nullptr;        // [hub_cap] tag of the launch each query's walk ended in
  // hub batching: the hub vertices and the buffers of a hub-batched call (grown on demand)
  int hub_mode = -1;           // -1: when it pays, 0: never, 1: whenever the graph has hubs, 2: as 1 without the tail launch
  struct HubSet {                  // the hub vertices for one limit
    int32_t n = 0;
    uint32_t limit = 0;            // a vertex is a hub iff its row has at least this many edges
    int32_t* d_ids = nullptr;      // ascending
    uint32_t* d_cnt = nullptr;     // [2][n * classes] parked walkers per hub and class, this round and the next
    uint32_t* d_base = nullptr;    // [n * classes]
    uint32_t* d_fill = nullptr;    // [n * classes]
    int classes_cap = 0;           // classes the three arrays above are sized for
    uint16_t* d_parts = nullptr;   // [n] parts the sweep of a hub's row is split into
    uint16_t* d_ones = nullptr;    // [n] the same for node2vec, whose hub kernel does not split rows
    uint64_t parts_total = 0;      // their sum
    double mean_degree = 0;        // mean row length of a hub
  } hubset[2];                     // 0: limit 1,016, 1: limit 504
  size_t hub_cap = 0;              // queries the buffers below are sized for
  int32_t* d_kstate = nullptr;
  int32_t* d_list = nullptr;
  int32_t* d_park_hub[2] = {nullptr, nullptr};
  int32_t* d_park_qi[2] = {nullptr, nullptr};
  int32_t* d_bucket = nullptr;
  int4* d_items = nullptr;
  size_t items_cap = 0;
  unsigned long long* d_best64 = nullptr;  // [hub_cap]
  uint32_t* d_part_done = nullptr;         // [items_cap]
  uint2* d_tile_tot = nullptr;     // plan: per tile of keys, walkers and items (then their offsets)
  unsigned char* d_ctl = nullptr;  // two HubCtl blocks
  uint32_t* h_ctl = nullptr;       // pinned word the parked count travels to
  // staging for the host-buffer entry points (grown on demand)
  int32_t* d_starts[2] = {nullptr, nullptr};
  int32_t* d_result[2] = {nullptr, nullptr};
  size_t cap_starts[2] = {0, 0}, cap_result[2] = {0, 0};
};

namespace {

#define FW_CUDA(call)                                                                   \
  do {                                                                                  \
    cudaError_t err__ = (call);                                                         \
    if (err__ != cudaSuccess)                                                           \
      return fw::fail(FW_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(err__));  \
  } while (0)

struct DeviceGuard {
  int prev = 0;
  bool ok = false;  // the requested device is current
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    int now = -1;
    ok = cudaSetDevice(dev) == cudaSuccess && cudaGetDevice(&now) == cudaSuccess && now == dev;
  }
  ~DeviceGuard() { cudaSetDevice(prev); }
};

// Edge arrays are padded to whole quads (plus one) so that 16-byte loads of
// the first and last quad of any row stay inside the allocation.
template <typename T>
int upload_edges(const T* host, int64_t E, T** out, int device, bool managed) {
  const size_t padded = ((size_t)E + 3) / 4 * 4 + 4;
  if (managed) {
    // Unified memory (the role of --umgraph, include/gpu_graph.cuh:46-54): the array may exceed
    // the device's memory; pages live on the device as far as they fit and migrate on demand.
    FW_CUDA(cudaMallocManaged(out, padded * sizeof(T)));
    FW_CUDA(cudaMemAdvise(*out, padded * sizeof(T), cudaMemAdviseSetPreferredLocation, device));
  } else {
    FW_CUDA(cudaMalloc(out, padded * sizeof(T)));
  }
  const size_t tail = (size_t)E / 4 * 4;  // the padding, and the last partial quad, start at zero
  FW_CUDA(cudaMemset(*out + tail, 0, (padded - tail) * sizeof(T)));
  if (E > 0) FW_CUDA(cudaMemcpy(*out, host, (size_t)E * sizeof(T), cudaMemcpyHostToDevice));
  if (managed) {
    size_t free_b = 0, total_b = 0;
    FW_CUDA(cudaMemGetInfo(&free_b, &total_b));
    const size_t keep = (size_t)1 << 30;  // leave room for results and the other arrays' share
    const size_t fit = free_b > keep ? std::min(padded * sizeof(T), free_b - keep) : 0;
    if (fit) FW_CUDA(cudaMemPrefetchAsync(*out, fit, device, 0));
    FW_CUDA(cudaDeviceSynchronize());
  }
  return FW_OK;
}

int ensure_scratch(fw_engine* e, int d) {
  const size_t words = (size_t)kSlotHist + (size_t)d + 1;
  if (words <= e->scratch_words) return FW_OK;
  if (e->d_scratch) cudaFree(e->d_scratch);
  if (e->h_scratch) cudaFreeHost(e->h_scratch);
  e->d_scratch = nullptr; e->h_scratch = nullptr; e->scratch_words = 0;
  const size_t cap = std::max<size_t>(words, 1024);
  FW_CUDA(cudaMalloc(&e->d_scratch, cap * 8));
  FW_CUDA(cudaMallocHost(&e->h_scratch, cap * 8));
  e->scratch_words = cap;
  return FW_OK;
}

int check_params(const fw_engine* e, const fw_walk_params* p, int64_t n) {
  if (!e || !p) return fw::fail(FW_ERR_ARG, "null engine or params");
  if (n < 0) return fw::fail(FW_ERR_ARG, "negative query count");
  if (p->app < FW_APP_DEEPWALK || p->app > FW_APP_METAPATH) return fw::fail(FW_ERR_ARG, "unknown app %d", p->app);
  if (p->d < 0 || p->d >= (1 << 28)) return fw::fail(FW_ERR_ARG, "d out of range");
  if (p->group_mode != 0 && p->group_mode != FW_GROUP_EDGE && p->group_mode != FW_GROUP_STRIP)
    return fw::fail(FW_ERR_ARG, "group_mode must be 0, %d or %d", FW_GROUP_EDGE, FW_GROUP_STRIP);
  if (p->app == FW_APP_METAPATH) {
    if (!e->d_label) return fw::fail(FW_ERR_ARG, "MetaPath needs edge labels on the device");
    if (!p->schema || p->schema_len <= 0 || p->schema_len > kMaxSchema)
      return fw::fail(FW_ERR_ARG, "schema length must be in 1..%d", kMaxSchema);
  } else if (!e->d_weight) {
    return fw::fail(FW_ERR_ARG, "this app needs edge weights on the device");
  }
  if (p->app == FW_APP_NODE2VEC && !(p->p > 0.0 && p->q > 0.0))
    return fw::fail(FW_ERR_ARG, "node2vec needs p > 0 and q > 0");
  return FW_OK;
}

// Lets `fn` use `smem` bytes of dynamic shared memory and returns how many of its CTAs fit on an
// SM.  Without the opt-in a kernel's dynamic and static shared memory together are limited to
// 48 KB, so the test counts the kernel's static part as well (the walk kernels hold their
// mbarriers, node2vec's match flags and the CTA's board there).
int prepare_kernel(KernelFn fn, size_t smem, int* per_sm) {
  cudaFuncAttributes attr;
  FW_CUDA(cudaFuncGetAttributes(&attr, (const void*)fn));
  if (smem + attr.sharedSizeBytes > 48 * 1024)
    FW_CUDA(cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  *per_sm = 0;
  FW_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(per_sm, fn, kThreads, smem));
  if (*per_sm < 1) return fw::fail(FW_ERR_CUDA, "walk kernel does not fit on an SM");
  return FW_OK;
}

// Enqueues: scratch reset, kernel between ev[0] and ev[1], scratch read-back.
// Buffers of a hub-batched call for n queries.
int ensure_hub_buffers(fw_engine* e, size_t n, size_t classes) {
  const size_t parts_total = (size_t)std::max(e->hubset[0].parts_total, e->hubset[1].parts_total) * classes;
  if (n <= e->hub_cap && (e->hub_cap / 32) * (size_t)kHubMaxParts + parts_total + 1 <= e->items_cap) return FW_OK;
  n = std::max(n, e->hub_cap);
  cudaFree(e->d_kstate); cudaFree(e->d_list); cudaFree(e->d_bucket); cudaFree(e->d_items);
  cudaFree(e->d_best64); cudaFree(e->d_part_done); cudaFree(e->d_fin);
  for (int i = 0; i < 2; ++i) { cudaFree(e->d_park_hub[i]); cudaFree(e->d_park_qi[i]); }
  e->d_kstate = e->d_list = e->d_bucket = e->d_fin = nullptr;
  e->d_items = nullptr; e->d_best64 = nullptr; e->d_part_done = nullptr;
  e->d_park_hub[0] = e->d_park_hub[1] = e->d_park_qi[0] = e->d_park_qi[1] = nullptr;
  e->hub_cap = 0;
  const size_t cap = std::max<size_t>(n, 1024);
  FW_CUDA(cudaMalloc(&e->d_kstate, cap * 4));
  FW_CUDA(cudaMalloc(&e->d_fin, cap * 4));
  FW_CUDA(cudaMalloc(&e->d_list, cap * 4));
  FW_CUDA(cudaMalloc(&e->d_bucket, cap * 4));
  for (int i = 0; i < 2; ++i) {
    FW_CUDA(cudaMalloc(&e->d_park_hub[i], cap * 4));
    FW_CUDA(cudaMalloc(&e->d_park_qi[i], cap * 4));
  }
  // every hub has at most one batch that is not full, every batch one item per part of the row
  e->items_cap = (cap / 32) * (size_t)kHubMaxParts + parts_total + 1;
  FW_CUDA(cudaMalloc(&e->d_items, e->items_cap * sizeof(int4)));
  FW_CUDA(cudaMalloc(&e->d_part_done, e->items_cap * 4));
  FW_CUDA(cudaMalloc(&e->d_best64, cap * 8));
  e->hub_cap = cap;
  return FW_OK;
}

// The launches of a hub-batched call (see hub_kernel): the walk kernel on the fresh queries, then
// rounds of plan, scatter, hub kernel, walk kernel while walkers are parked at hubs.  Every round
// ends with the host reading the number of parked walkers, so this returns with the walk done.
int run_hub_batched(fw_engine* e, fw_engine::HubSet& hs, const fw_walk_params* p, WalkArgs a, int64_t n,
                    cudaStream_t st, size_t smem, int32_t* host_table, bool* table_delivered, int* launches) {
  *table_delivered = false;
  // rows shorter than a 128-byte segment are not worth a warp each: such tables travel in one copy
  if (p->d + 1 < kDeliverMinCells) host_table = nullptr;
  // MetaPath: walkers at the same step modulo the schema length want the same label and may share a sweep
  const int classes = p->app == FW_APP_METAPATH ? p->schema_len : 1;
  const size_t keys = (size_t)hs.n * (size_t)classes;
  int rc = ensure_hub_buffers(e, (size_t)n, (size_t)classes);
  if (rc) return rc;
  if (classes > hs.classes_cap) {
    cudaFree(hs.d_cnt); cudaFree(hs.d_base); cudaFree(hs.d_fill);
    hs.d_cnt = hs.d_base = hs.d_fill = nullptr;
    hs.classes_cap = 0;
    FW_CUDA(cudaMalloc(&hs.d_cnt, keys * 8));
    FW_CUDA(cudaMalloc(&hs.d_base, keys * 4));
    FW_CUDA(cudaMalloc(&hs.d_fill, keys * 4));
    hs.classes_cap = classes;
  }
  KernelFn walk_fn = pick_hub_kernel(p->app, hs.limit == kHubLimitLow ? 3 : 0, e->clean_weights, e->xadj_bits);
  KernelFn hub_fn = pick_hub_kernel(p->app, 1, e->clean_weights, e->xadj_bits);
  KernelFn tail_fn = pick_hub_kernel(p->app, 2, e->clean_weights, e->xadj_bits);
  int walk_per_sm = 0, hub_per_sm = 0, tail_per_sm = 0;
  // node2vec's walk kernels keep their own ring; its hub kernel sweeps like the others'
  const bool n2v = p->app == FW_APP_NODE2VEC;
  const size_t walk_smem = n2v ? smem : hub_walk_smem_bytes(hs.limit, p->d, a.hist_in_smem != 0);
  const size_t hub_smem = kernel_smem_bytes(FW_APP_DEEPWALK, FW_GROUP_STRIP, p->d, a.hist_in_smem != 0);
  const uint16_t* d_parts = n2v ? hs.d_ones : hs.d_parts;
  rc = prepare_kernel(walk_fn, walk_smem, &walk_per_sm);
  if (!rc) rc = prepare_kernel(hub_fn, hub_smem, &hub_per_sm);
  if (!rc) rc = prepare_kernel(tail_fn, smem, &tail_per_sm);
  if (rc) return rc;
  // Below this many parked walkers the batches are mostly empty and a round costs more than it
  // serves: the walkers left are then walked to the end by one launch, each sweeping for itself.
  const char* te_env = getenv("FW_HUB_TAIL_EDGES");  // development aid
  const double tail_edges = te_env && atof(te_env) > 0 ? atof(te_env) : kHubTailEdges;
  const uint32_t tail_limit = e->hub_mode == 2 ? 0u
      : (uint32_t)std::max<double>((double)kHubTailMin, std::min<double>(tail_edges / hs.mean_degree, (double)n / 4));
  HubCtl* ctl = reinterpret_cast<HubCtl*>(e->d_ctl);
  FW_CUDA(cudaMemsetAsync(e->d_ctl, 0, 2 * sizeof(HubCtl), st));
  FW_CUDA(cudaMemsetAsync(hs.d_cnt, 0, keys * 8, st));
  a.hub.hub_ids = hs.d_ids; a.hub.n_hubs = hs.n; a.hub.min_degree = hs.limit; a.hub.classes = classes;
  a.hub.kstate = e->d_kstate;
  a.hub.next_list = e->d_list; a.hub.bucket = e->d_bucket; a.hub.items = e->d_items;
  a.hub.hub_parts = d_parts; a.hub.best64 = e->d_best64; a.hub.part_done = e->d_part_done;
  // Early delivery: rows of walks that ended up to the launches enqueued so far go to the caller's
  // host table on a stream of their own, behind an event on the walk stream.  d_fin serves one call
  // at a time: the walk stream waits for the previous call's last delivery before it clears it.
  // The device's stores over PCIe are slower than the copy engine (45 against 57 GB/s alone, about
  // 20 GB/s beside the walk kernels, which they slow by a tenth), so delivery pays only where the
  // walk lasts about as long as the copy would: it begins once the series has run for a quarter of
  // the time the table needs on the link (a call that is over before then copies the table in one
  // piece, as without delivery), and a call that ends with less than a quarter of its rows delivered
  // stops the launches in flight and copies the whole table as well.
  int32_t tag = 0, delivered_to = 0;
  bool delivering = false;
  const int deliver_grid = [&] {
    const char* env = getenv("FW_DELIVER_CTAS");  // development aid
    return env && atoi(env) > 0 ? atoi(env) : kDeliverCtas;
  }();
  DeliverCtl* const dctl = reinterpret_cast<DeliverCtl*>(e->d_ctl + 2 * sizeof(HubCtl));
  const double link_us = (double)n * (double)(p->d + 1) * 4.0 / kLinkBytesPerUs;
  const auto t_begin = std::chrono::steady_clock::now();
  if (host_table) {
    FW_CUDA(cudaStreamWaitEvent(st, e->ev_out, 0));
    FW_CUDA(cudaMemsetAsync(e->d_fin, 0, (size_t)n * 4, st));
    FW_CUDA(cudaMemsetAsync(dctl, 0, sizeof(DeliverCtl), st));
    a.hub.fin = e->d_fin;
  }
  // after the launches of a round have been enqueued
  auto deliver = [&]() -> int {
    if (!host_table) return FW_OK;
    if (!delivering) {
      const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t_begin).count();
      if (e->early_delivery < 1 && us < link_us / 4) return FW_OK;
      delivering = true;
    }
    FW_CUDA(cudaEventRecord(e->ev_round, st));
    FW_CUDA(cudaStreamWaitEvent(e->stream_out, e->ev_round, 0));
    deliver_kernel<<<deliver_grid, kDeliverThreads, 0, e->stream_out>>>(a.result, host_table, e->d_fin, (long long)n, p->d + 1,
                                                                         delivered_to, tag, dctl);
    FW_CUDA(cudaGetLastError());
    delivered_to = tag;
    ++*launches;
    return FW_OK;
  };
  // when the last launch of the series has returned: the rest of the table, one way or the other
  auto finish_delivery = [&]() -> int {
    if (!host_table || !delivering) return FW_OK;
    FW_CUDA(cudaMemcpyAsync(e->h_ctl + 2, &dctl->rows, 4, cudaMemcpyDeviceToHost, st));
    FW_CUDA(cudaStreamSynchronize(st));
    if (e->early_delivery == 2 || (e->early_delivery < 1 && (int64_t)e->h_ctl[2] < n / 4)) {
      FW_CUDA(cudaMemsetAsync(&dctl->stop, 0xFF, 4, st));
    } else {
      deliver_kernel<<<deliver_grid, kDeliverThreads, 0, e->stream_out>>>(a.result, host_table, e->d_fin, (long long)n, p->d + 1,
                                                                           delivered_to, INT32_MAX, dctl);
      FW_CUDA(cudaGetLastError());
      ++*launches;
      *table_delivered = true;
    }
    FW_CUDA(cudaEventRecord(e->ev_out, e->stream_out));  // the caller's stream waits for this one
    return FW_OK;
  };
  auto parks_into = [&](int set) {
    a.hub.park_hub = e->d_park_hub[set]; a.hub.park_qi = e->d_park_qi[set];
    a.hub.park_n = &ctl[set].park_n; a.hub.hub_cnt = hs.d_cnt + (size_t)set * keys;
  };
  void* params[] = {&a};
  const int full_walk = e->sms * walk_per_sm, full_hub = e->sms * hub_per_sm;
  // the fresh queries
  int cur = 0;
  parks_into(cur);
  a.hub.list = nullptr; a.hub.list_n = nullptr; a.hub.work = &ctl[cur].work_walk;
  {
    const int64_t want = (n + (kThreads / 32) * kMinClaim - 1) / ((kThreads / 32) * kMinClaim);
    const int grid = (int)std::min<int64_t>(full_walk, std::max<int64_t>(want, 1));
    a.hub.fin_tag = ++tag;
    FW_CUDA(cudaLaunchKernel((const void*)walk_fn, dim3(grid), dim3(kThreads), params, walk_smem, st));
    ++*launches;
    rc = deliver();
    if (rc) return rc;
  }
  const bool trace = getenv("FW_HUB_TRACE") != nullptr;  // development aid: the rounds on stderr
  const auto t_trace = std::chrono::steady_clock::now();
  // every round moves each parked walker at least one step on: d + 1 rounds are the most there can be
  for (int64_t round = 0;; ++round) {
    FW_CUDA(cudaMemcpyAsync(e->h_ctl, &ctl[cur].park_n, 4, cudaMemcpyDeviceToHost, st));
    FW_CUDA(cudaStreamSynchronize(st));
    const uint32_t parked = e->h_ctl[0];
    if (trace) {
      const double now = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t_trace).count();
      fprintf(stderr, "hub round %lld: %u parked, %.0f us since the call began\n", (long long)round, parked, now);
    }
    if (parked == 0) break;
    if (parked < tail_limit) {
      a.hub.list = e->d_park_qi[cur]; a.hub.list_n = &ctl[cur].park_n; a.hub.work = &ctl[cur].work_hub;
      const int tgrid = (int)std::min<int64_t>((int64_t)e->sms * tail_per_sm, std::max<int64_t>(((int64_t)parked + 31) / 32, 1));
      a.hub.fin_tag = ++tag;
      FW_CUDA(cudaLaunchKernel((const void*)tail_fn, dim3(tgrid), dim3(kThreads), params, smem, st));
      ++*launches;
      // the engine's hub buffers serve one call at a time: the next one (a batch on the other
      // stream) may start only when this launch is through with them
      FW_CUDA(cudaStreamSynchronize(st));
      break;
    }
    if (round > (int64_t)p->d + 1) return fw::fail(FW_ERR_DEVICE, "hub batching did not come to an end (internal error)");
    const int nxt = cur ^ 1;
    FW_CUDA(cudaMemsetAsync(&ctl[nxt], 0, sizeof(HubCtl), st));
    FW_CUDA(cudaMemsetAsync(e->d_best64, 0xFF, (size_t)parked * 8, st));
    const int tiles = (int)((keys + kPlanTile - 1) / kPlanTile);
    hub_plan_count<<<tiles, kPlanThreads, 0, st>>>(hs.d_cnt + (size_t)cur * keys, d_parts, (int)keys, classes, e->d_tile_tot,
                                                   &ctl[cur].tiles_done, &ctl[cur].items_n);
    hub_plan_emit<<<tiles, kPlanThreads, 0, st>>>(hs.d_cnt + (size_t)cur * keys, hs.d_base, hs.d_fill, e->d_items, d_parts,
                                                  e->d_part_done, (int)keys, classes, e->d_tile_tot);
    const int sgrid = (int)std::min<int64_t>(((int64_t)parked + 255) / 256, (int64_t)e->sms * 8);
    hub_scatter_kernel<<<sgrid, 256, 0, st>>>(e->d_park_hub[cur], e->d_park_qi[cur], &ctl[cur].park_n, hs.d_base, hs.d_fill,
                                              e->d_bucket);
    FW_CUDA(cudaGetLastError());
    // hub kernel: serves this round's batches, parks and lists for the next
    parks_into(nxt);
    a.hub.items_n = &ctl[cur].items_n; a.hub.work = &ctl[cur].work_hub; a.hub.next_n = &ctl[nxt].list_n;
    a.hub.list = nullptr; a.hub.list_n = nullptr;
    const int64_t max_items = ((int64_t)parked / 32) * kHubMaxParts + (int64_t)hs.parts_total * classes;
    const int hgrid = (int)std::min<int64_t>(full_hub, std::max<int64_t>((max_items + 7) / 8, 1));
    a.hub.fin_tag = ++tag;
    FW_CUDA(cudaLaunchKernel((const void*)hub_fn, dim3(hgrid), dim3(kThreads), params, hub_smem, st));
    // walk kernel: the walkers the hub kernel listed
    a.hub.list = e->d_list; a.hub.list_n = &ctl[nxt].list_n; a.hub.work = &ctl[nxt].work_walk;
    const int wgrid = (int)std::min<int64_t>(full_walk, std::max<int64_t>(((int64_t)parked + 31) / 32, 1));
    FW_CUDA(cudaLaunchKernel((const void*)walk_fn, dim3(wgrid), dim3(kThreads), params, walk_smem, st));
    *launches += 5;
    cur = nxt;
    rc = deliver();
    if (rc) return rc;
  }
  return finish_delivery();
}

// The device's view of `bytes` of host memory at `host`, if all of it is page-locked memory the
// device can address (cudaHostAlloc, cudaMallocHost, cudaHostRegister); nullptr otherwise.
int32_t* device_view(const fw_engine* e, const void* host, size_t bytes) {
  if (e->early_delivery == 0 || !host || bytes == 0) return nullptr;
  const char* env = getenv("FLOWWALKER_EARLY_DELIVERY");
  if (env && env[0] == '0') return nullptr;
  cudaPointerAttributes first, last;
  if (cudaPointerGetAttributes(&first, host) != cudaSuccess ||
      cudaPointerGetAttributes(&last, static_cast<const char*>(host) + bytes - 1) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (first.type != cudaMemoryTypeHost || last.type != cudaMemoryTypeHost || !first.devicePointer || !last.devicePointer)
    return nullptr;
  if (static_cast<char*>(last.devicePointer) - static_cast<char*>(first.devicePointer) != (ptrdiff_t)(bytes - 1)) return nullptr;
  return static_cast<int32_t*>(first.devicePointer);
}

// Enqueues: scratch reset, kernel(s) between ev_begin and ev_end, scratch read-back.  *launches
// receives the number of kernel launches.  A hub-batched call has returned from its last kernel
// when this returns; a single-kernel call is only enqueued.
int enqueue_walk(fw_engine* e, const fw_walk_params* p, const int32_t* starts_dev, int64_t n,
                 int32_t* result_dev, cudaStream_t st, cudaEvent_t ev_begin, cudaEvent_t ev_end,
                 unsigned long long* d_scratch, unsigned long long* h_scratch, int* launches,
                 int32_t* host_table = nullptr, bool* delivered = nullptr) {
  *launches = 0;
  if (delivered) *delivered = false;
  WalkArgs a;
  memset(&a.hub, 0, sizeof(a.hub));
  a.xadj = e->d_xadj; a.adj = e->d_adj; a.weight = e->d_weight; a.label = e->d_label;
  a.V = e->V; a.starts = starts_dev; a.n = n; a.result = result_dev; a.scratch = d_scratch;
  a.qid_base = p->query_id_base; a.qid_stride = p->query_id_stride ? p->query_id_stride : 1; a.d = p->d;
  a.tp_thresh = fw::tp_threshold(p->tp);
  a.inv_p = (float)(1.0 / p->p); a.inv_q = (float)(1.0 / p->q);
  a.n2v_fmax = std::max(1.0f, std::max(a.inv_p, a.inv_q)) * 1.00001f;
  a.k0 = (uint32_t)p->seed; a.k1 = (uint32_t)(p->seed >> 32);
  fw::philox_round_keys(a.k0, a.k1, a.rk);
  a.hist_in_smem = p->d + 1 <= kMaxSmemHist;
  a.schema_len = p->app == FW_APP_METAPATH ? p->schema_len : 1;
  for (int i = 0; i < kMaxSchema; ++i) a.schema[i] = (p->app == FW_APP_METAPATH && i < p->schema_len) ? p->schema[i] : 0;
  const int mode = p->group_mode == 0 ? FW_GROUP_STRIP : p->group_mode;
  // measured: sharing halves DeepWalk's time on a graph with 10^6-edge hubs (2012 -> 974 ms) and
  // costs node2vec 20 % there (its shared variant spills), so node2vec shares only on request
  const bool shared = e->sharing > 0 ||
                      (e->sharing < 0 && p->app != FW_APP_NODE2VEC && e->max_degree >= kSharingAutoDegree);
  KernelFn fn = pick_kernel(p->app, mode, e->clean_weights, shared, e->xadj_bits);
  const size_t smem = kernel_smem_bytes(p->app, mode, p->d, a.hist_in_smem != 0);
  int per_sm = 0;
  const int prc = prepare_kernel(fn, smem, &per_sm);
  if (prc) return prc;
  const size_t words = (size_t)kSlotHist + (size_t)p->d + 1;
  FW_CUDA(cudaMemsetAsync(d_scratch, 0, words * 8, st));
  FW_CUDA(cudaEventRecord(ev_begin, st));
  // Hub batching, with the strip sampler on graphs that have hub vertices: the strip totals of a row
  // do not depend on the walker (MetaPath: on the label it wants; node2vec: the plain totals its
  // sweep forms).  Query and vertex numbers must fit 31 bits.
  // The lower hub limit when the call brings enough queries per hub to fill the batches.
  // (node2vec: the higher limit always; its walk kernel stages nothing)
  fw_engine::HubSet& hs = (p->app != FW_APP_NODE2VEC && e->hubset[1].n > 0 && n >= kHubDenseQueries * e->hubset[1].n)
                              ? e->hubset[1] : e->hubset[0];
  const bool worth_it = e->hub_mode > 0 || n >= kHubMinQueries * (int64_t)e->hubset[0].n;
  const bool hubs = e->hub_mode != 0 && worth_it && hs.n > 0 && mode == FW_GROUP_STRIP && e->sharing <= 0 &&
                    n < ((int64_t)1 << 31) &&
                    (int64_t)hs.n * (p->app == FW_APP_METAPATH ? p->schema_len : 1) <= (int64_t)kPlanMaxTiles * kPlanTile / 2;
  if (n > 0 && hubs) {
    bool table_delivered = false;
    const int hrc = run_hub_batched(e, hs, p, a, n, st, smem, host_table, &table_delivered, launches);
    if (hrc) return hrc;
    if (delivered) *delivered = table_delivered;
  } else if (n > 0) {
    const int64_t want = (n + (kThreads / 32) * kMinClaim - 1) / ((kThreads / 32) * kMinClaim);
    const int grid = (int)std::min<int64_t>((int64_t)e->sms * per_sm, std::max<int64_t>(want, 1));
    void* params[] = {&a};
    FW_CUDA(cudaLaunchKernel((const void*)fn, dim3(grid), dim3(kThreads), params, smem, st));
    *launches = 1;
  }
  FW_CUDA(cudaEventRecord(ev_end, st));
  if (host_table && n > 0 && hubs) FW_CUDA(cudaStreamWaitEvent(st, e->ev_out, 0));  // the table is complete when st is
  FW_CUDA(cudaMemcpyAsync(h_scratch, d_scratch, words * 8, cudaMemcpyDeviceToHost, st));
  return FW_OK;
}

// Returns FW_ERR_DEVICE when the kernel gave up on a bounded wait (the walks of that launch are
// incomplete); bad start or neighbour ids only set their status bits.
int collect(const unsigned long long* h, int d, float ms, int launches, fw_walk_stats* stats,
            uint64_t* len_hist, bool accumulate) {
  if (stats) {
    if (!accumulate) { stats->steps = 0; stats->scanned = 0; stats->device_ms = 0; stats->device_status = 0; stats->launches = 0; }
    stats->steps += h[kSlotSteps];
    stats->scanned += h[kSlotScanned];
    stats->device_status |= (uint32_t)h[kSlotStatus];
    stats->device_ms += ms;
    stats->launches += (uint32_t)launches;
  }
  if (len_hist)
    for (int z = 0; z <= d; ++z) len_hist[z] = (accumulate ? len_hist[z] : 0) + h[kSlotHist + z];
  if (h[kSlotStatus] & FW_STATUS_WAIT_TIMEOUT)
    return fw::fail(FW_ERR_DEVICE, "the walk kernel gave up waiting for a staged copy; the result is incomplete");
  return FW_OK;
}

template <typename T>
int ensure_cap(T** buf, size_t* cap, size_t need) {
  if (need <= *cap) return FW_OK;
  if (*buf) cudaFree(*buf);
  *buf = nullptr; *cap = 0;
  cudaError_t err = cudaMalloc(buf, std::max<size_t>(need, 1) * sizeof(T));
  if (err != cudaSuccess)
    return fw::fail(FW_ERR_NOMEM, "cudaMalloc of %zu bytes failed: %s", need * sizeof(T), cudaGetErrorString(err));
  *cap = need;
  return FW_OK;
}

}  // namespace

extern "C" const char* fw_kernel_revision(void) { return FW_KERNEL_REVISION; }

extern "C" int fw_device_count(int* count) {
  fw::clear_error();
  if (!count) return fw::fail(FW_ERR_ARG, "fw_device_count: null argument");
  *count = 0;
  cudaError_t err = cudaGetDeviceCount(count);
  if (err == cudaErrorNoDevice || err == cudaErrorInsufficientDriver) { *count = 0; return FW_OK; }
  if (err != cudaSuccess) return fw::fail(FW_ERR_CUDA, "cudaGetDeviceCount failed: %s", cudaGetErrorString(err));
  return FW_OK;
}

extern "C" int fw_engine_create(const fw_graph* g, int device, int which, fw_engine** out) {
  fw::clear_error();
  if (!g || !out) return fw::fail(FW_ERR_ARG, "fw_engine_create: null argument");
  *out = nullptr;
  int count = 0;
  FW_CUDA(cudaGetDeviceCount(&count));
  if (device < 0 || device >= count) return fw::fail(FW_ERR_ARG, "device %d out of range (%d visible)", device, count);
  DeviceGuard guard(device);
  cudaDeviceProp prop;
  FW_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major < 10) return fw::fail(FW_ERR_CUDA, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
  fw_engine* e = new (std::nothrow) fw_engine();
  if (!e) return fw::fail(FW_ERR_NOMEM, "out of host memory");
  e->device = device; e->sms = prop.multiProcessorCount;
  e->V = g->V; e->E = g->E; e->xadj_bits = g->xadj_bits;
  const bool managed = (which & FW_ENGINE_MANAGED) != 0;
  which &= ~FW_ENGINE_MANAGED;
  if (which < 0 || which > 3) { delete e; return fw::fail(FW_ERR_ARG, "fw_engine_create: unknown bits in `which`"); }
  const bool want_w = which == 0 ? g->weight != nullptr : (which & 1) != 0;
  const bool want_l = which == 0 ? g->label != nullptr : (which & 2) != 0;
  int rc = FW_OK;
  auto body = [&]() -> int {
    for (int64_t v = 0; v < g->V; ++v)
      e->max_degree = std::max(e->max_degree, fw::row_begin(g, v + 1) - fw::row_begin(g, v));
    // Hubs: every vertex of at least `limit` neighbours, for both limits (the walk kernel of a
    // hub-batched call relies on every other row fitting one stage); a graph with more than
    // kHubMax of them runs without hub batching at that limit.
    const char* ps_env = getenv("FW_HUB_PART_SUPERS");  // development aid
    const int64_t part_supers = ps_env && atoll(ps_env) > 0 ? atoll(ps_env) : kHubPartSupers;
    for (int which = 0; which < 2 && g->V < INT32_MAX; ++which) {
      fw_engine::HubSet& hs = e->hubset[which];
      const int64_t limit = which ? kHubLimitLow : kHubLimitHigh;
      std::vector<int32_t> ids;
      for (int64_t v = 0; v < g->V && (int64_t)ids.size() <= kHubMax; ++v)
        if (fw::row_begin(g, v + 1) - fw::row_begin(g, v) >= limit) ids.push_back((int32_t)v);
      if (ids.empty() || (int64_t)ids.size() > kHubMax) continue;
      // rows of more than kHubPartSupers supergroups are swept by several warps, a part each
      std::vector<uint16_t> parts(ids.size());
      double sum_len = 0;
      for (size_t i = 0; i < ids.size(); ++i) {
        const int64_t b = fw::row_begin(g, ids[i]), len = fw::row_begin(g, (int64_t)ids[i] + 1) - b;
        sum_len += (double)len;
        const int64_t nq = ((b & 3) + len + 3) >> 2, n_half = (nq + kHalfQuads - 1) / kHalfQuads, supers = (n_half + 1) >> 1;
        parts[i] = (uint16_t)std::min<int64_t>(kHubMaxParts, (supers + part_supers - 1) / part_supers);
        hs.parts_total += parts[i];
      }
      hs.n = (int32_t)ids.size();
      hs.limit = (uint32_t)limit;
      hs.mean_degree = sum_len / (double)ids.size();
      FW_CUDA(cudaMalloc(&hs.d_ids, ids.size() * 4));
      FW_CUDA(cudaMemcpy(hs.d_ids, ids.data(), ids.size() * 4, cudaMemcpyHostToDevice));
      FW_CUDA(cudaMalloc(&hs.d_parts, parts.size() * 2));
      FW_CUDA(cudaMemcpy(hs.d_parts, parts.data(), parts.size() * 2, cudaMemcpyHostToDevice));
      std::fill(parts.begin(), parts.end(), (uint16_t)1);
      FW_CUDA(cudaMalloc(&hs.d_ones, parts.size() * 2));
      FW_CUDA(cudaMemcpy(hs.d_ones, parts.data(), parts.size() * 2, cudaMemcpyHostToDevice));
    }
    if (e->hubset[0].n > 0 || e->hubset[1].n > 0) {
      FW_CUDA(cudaMalloc(&e->d_tile_tot, (size_t)kPlanMaxTiles * sizeof(uint2)));
      FW_CUDA(cudaMalloc(&e->d_ctl, 2 * sizeof(HubCtl) + sizeof(DeliverCtl)));
      FW_CUDA(cudaMallocHost(&e->h_ctl, 64));
    }
    if (want_w && !g->weight) return fw::fail(FW_ERR_ARG, "graph has no weights");
    if (want_l && !g->label) return fw::fail(FW_ERR_ARG, "graph has no labels");
    const size_t xb = (size_t)(g->xadj_bits / 8) * (size_t)(g->V + 2);
    FW_CUDA(cudaMalloc(&e->d_xadj, xb));
    FW_CUDA(cudaMemcpy(e->d_xadj, g->xadj, (size_t)(g->xadj_bits / 8) * (size_t)(g->V + 1), cudaMemcpyHostToDevice));
    int r = upload_edges(g->adj, g->E, &e->d_adj, device, managed);
    if (!r && want_w) r = upload_edges(g->weight, g->E, &e->d_weight, device, managed);
    if (want_w) {
      bool clean = true;
      for (int64_t i = 0; i < g->E && clean; ++i) clean = g->weight[i] >= 0.0f;
      e->clean_weights = clean;
    }
    if (!r && want_l) r = upload_edges(g->label, g->E, &e->d_label, device, managed);
    if (r) return r;
    FW_CUDA(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
    FW_CUDA(cudaStreamCreateWithFlags(&e->stream2, cudaStreamNonBlocking));
    for (auto& ev : e->ev) FW_CUDA(cudaEventCreate(&ev));
    {
      // the delivery stream's few CTAs must not queue behind the walk kernels' full grids
      int prio_low = 0, prio_high = 0;
      FW_CUDA(cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high));
      FW_CUDA(cudaStreamCreateWithPriority(&e->stream_out, cudaStreamNonBlocking, prio_high));
      FW_CUDA(cudaEventCreateWithFlags(&e->ev_round, cudaEventDisableTiming));
      FW_CUDA(cudaEventCreateWithFlags(&e->ev_out, cudaEventDisableTiming));
    }
    return ensure_scratch(e, 1023);
  };
  rc = body();
  if (rc) { fw_engine_destroy(e); return rc; }
  *out = e;
  return FW_OK;
}

extern "C" void fw_engine_destroy(fw_engine* e) {
  if (!e) return;
  DeviceGuard guard(e->device);
  cudaFree(e->d_xadj); cudaFree(e->d_adj); cudaFree(e->d_weight); cudaFree(e->d_label);
  cudaFree(e->d_scratch);
  if (e->h_scratch) cudaFreeHost(e->h_scratch);
  for (auto& hs : e->hubset) { cudaFree(hs.d_ids); cudaFree(hs.d_cnt); cudaFree(hs.d_base); cudaFree(hs.d_fill); cudaFree(hs.d_parts); cudaFree(hs.d_ones); }
  cudaFree(e->d_ctl); cudaFree(e->d_tile_tot);
  if (e->h_ctl) cudaFreeHost(e->h_ctl);
  cudaFree(e->d_kstate); cudaFree(e->d_list); cudaFree(e->d_bucket); cudaFree(e->d_items);
  cudaFree(e->d_best64); cudaFree(e->d_part_done); cudaFree(e->d_fin);
  for (int i = 0; i < 2; ++i) { cudaFree(e->d_park_hub[i]); cudaFree(e->d_park_qi[i]); }
  for (int i = 0; i < 2; ++i) { cudaFree(e->d_starts[i]); cudaFree(e->d_result[i]); }
  if (e->stream) cudaStreamDestroy(e->stream);
  if (e->stream2) cudaStreamDestroy(e->stream2);
  if (e->stream_out) cudaStreamDestroy(e->stream_out);
  for (auto& ev : e->ev) if (ev) cudaEventDestroy(ev);
  if (e->ev_round) cudaEventDestroy(e->ev_round);
  if (e->ev_out) cudaEventDestroy(e->ev_out);
  delete e;
}

extern "C" int fw_engine_set_sharing(fw_engine* e, int mode) {
  if (!e || mode < -1 || mode > 1) return fw::fail(FW_ERR_ARG, "fw_engine_set_sharing: mode must be -1, 0 or 1");
  e->sharing = mode;
  return FW_OK;
}

extern "C" int fw_engine_set_hub_batching(fw_engine* e, int mode) {
  if (!e || mode < -1 || mode > 2) return fw::fail(FW_ERR_ARG, "fw_engine_set_hub_batching: mode must be -1, 0, 1 or 2");
  e->hub_mode = mode;
  return FW_OK;
}

extern "C" int fw_engine_set_early_delivery(fw_engine* e, int mode) {
  if (!e || mode < -1 || mode > 2) return fw::fail(FW_ERR_ARG, "fw_engine_set_early_delivery: mode must be -1, 0, 1 or 2");
  e->early_delivery = mode;
  return FW_OK;
}

extern "C" int fw_engine_hubs(const fw_engine* e, int which, int32_t* n_hubs, uint32_t* min_degree) {
  if (!e || which < 0 || which > 1) return fw::fail(FW_ERR_ARG, "fw_engine_hubs: null engine or which not 0 / 1");
  if (n_hubs) *n_hubs = e->hubset[which].n;
  if (min_degree) *min_degree = which ? kHubLimitLow : kHubLimitHigh;
  return FW_OK;
}

extern "C" int fw_engine_device(const fw_engine* e, int* device, int* sm_count) {
  if (!e) return fw::fail(FW_ERR_ARG, "fw_engine_device: null engine");
  if (device) *device = e->device;
  if (sm_count) *sm_count = e->sms;
  return FW_OK;
}

extern "C" int fw_walk_device(fw_engine* e, const fw_walk_params* p, const int32_t* starts_dev,
                              int64_t n, int32_t* result_dev, void* stream, fw_walk_stats* stats,
                              uint64_t* len_hist) {
  fw::clear_error();
  int rc = check_params(e, p, n);
  if (rc) return rc;
  if (n > 0 && (!starts_dev || !result_dev)) return fw::fail(FW_ERR_ARG, "null device buffer");
  std::lock_guard<std::mutex> lock(e->mu);
  DeviceGuard guard(e->device);
  rc = ensure_scratch(e, p->d);
  if (rc) return rc;
  cudaStream_t st = stream ? (cudaStream_t)stream : e->stream;
  int launches = 0;
  rc = enqueue_walk(e, p, starts_dev, n, result_dev, st, e->ev[0], e->ev[1], e->d_scratch, e->h_scratch, &launches);
  if (rc) return rc;
  FW_CUDA(cudaStreamSynchronize(st));
  float ms = 0.f;
  FW_CUDA(cudaEventElapsedTime(&ms, e->ev[0], e->ev[1]));
  rc = collect(e->h_scratch, p->d, ms, launches, stats, len_hist, false);
  if (stats) stats->total_ms = ms;
  return rc;
}

extern "C" int fw_walk(fw_engine* e, const fw_walk_params* p, const int32_t* starts_host, int64_t n,
                       int32_t* result_host, fw_walk_stats* stats, uint64_t* len_hist) {
  fw::clear_error();
  int rc = check_params(e, p, n);
  if (rc) return rc;
  if (n > 0 && (!starts_host || !result_host)) return fw::fail(FW_ERR_ARG, "null host buffer");
  std::lock_guard<std::mutex> lock(e->mu);
  DeviceGuard guard(e->device);
  rc = ensure_scratch(e, p->d);
  if (rc) return rc;
  const size_t cells = (size_t)n * (size_t)(p->d + 1);
  rc = ensure_cap(&e->d_starts[0], &e->cap_starts[0], (size_t)n);
  if (!rc) rc = ensure_cap(&e->d_result[0], &e->cap_result[0], cells);
  if (rc) return rc;
  cudaStream_t st = e->stream;
  FW_CUDA(cudaEventRecord(e->ev[2], st));
  if (n > 0) FW_CUDA(cudaMemcpyAsync(e->d_starts[0], starts_host, (size_t)n * 4, cudaMemcpyHostToDevice, st));
  int launches = 0;
  bool delivered = false;
  rc = enqueue_walk(e, p, e->d_starts[0], n, e->d_result[0], st, e->ev[0], e->ev[1], e->d_scratch, e->h_scratch, &launches,
                    device_view(e, result_host, cells * 4), &delivered);
  if (rc) return rc;
  if (n > 0 && !delivered) FW_CUDA(cudaMemcpyAsync(result_host, e->d_result[0], cells * 4, cudaMemcpyDeviceToHost, st));
  FW_CUDA(cudaEventRecord(e->ev[3], st));
  FW_CUDA(cudaStreamSynchronize(st));
  float ms = 0.f, total = 0.f;
  FW_CUDA(cudaEventElapsedTime(&ms, e->ev[0], e->ev[1]));
  FW_CUDA(cudaEventElapsedTime(&total, e->ev[2], e->ev[3]));
  rc = collect(e->h_scratch, p->d, ms, launches, stats, len_hist, false);
  if (stats) stats->total_ms = total;
  return rc;
}

extern "C" void fw_free_pinned(void* p) {
  if (p) cudaFreeHost(p);
}

// Two streams, double-buffered batches (src/walk.cu:373-466): batch i+1 walks while the result of
// batch i travels to `pinned` (host memory of n*(d+1) cells, ideally page-locked).
static int walk_batches(fw_engine* e, const fw_walk_params* p, const int32_t* starts_host, int64_t n,
                        int64_t batch_size, int32_t headroom_mb, int32_t* pinned, fw_walk_stats* stats,
                        uint64_t* len_hist) {
  int rc = FW_OK;
  std::lock_guard<std::mutex> lock(e->mu);
  DeviceGuard guard(e->device);
  const size_t D = (size_t)p->d + 1;
  if (batch_size <= 0) {  // --autobatch, src/main.cu:259-271
    size_t free_b = 0, total_b = 0;
    FW_CUDA(cudaMemGetInfo(&free_b, &total_b));
    for (int i = 0; i < 2; ++i) free_b += e->cap_starts[i] * 4 + e->cap_result[i] * 4;
    const size_t head = (size_t)std::max(headroom_mb, 0) << 20;
    if (free_b <= head) return fw::fail(FW_ERR_NOMEM, "no device memory left after %d MB headroom", headroom_mb);
    batch_size = (int64_t)std::min<size_t>((free_b - head) / (4 * (D + 1)) / 2, (size_t)INT32_MAX);
    if (batch_size < 1) return fw::fail(FW_ERR_NOMEM, "device memory too small for one query");
  }
  batch_size = std::max<int64_t>(1, std::min(batch_size, std::max<int64_t>(n, 1)));
  // second scratch block for the second stream lives behind the first
  const size_t words = (size_t)kSlotHist + D;
  rc = ensure_scratch(e, (int)(2 * words));
  if (rc) return rc;
  auto bail = [&](int code) { cudaStreamSynchronize(e->stream); cudaStreamSynchronize(e->stream2); cudaStreamSynchronize(e->stream_out); return code; };
  for (int i = 0; i < 2; ++i) {
    rc = ensure_cap(&e->d_starts[i], &e->cap_starts[i], (size_t)batch_size);
    if (!rc) rc = ensure_cap(&e->d_result[i], &e->cap_result[i], (size_t)batch_size * D);
    if (rc) return bail(rc);
  }
  cudaStream_t streams[2] = {e->stream, e->stream2};
  cudaEvent_t evs[2][2] = {{e->ev[0], e->ev[1]}, {e->ev[2], e->ev[3]}};
  unsigned long long* dsc[2] = {e->d_scratch, e->d_scratch + words};
  unsigned long long* hsc[2] = {e->h_scratch, e->h_scratch + words};
  if (stats) { stats->steps = 0; stats->scanned = 0; stats->device_ms = 0; stats->total_ms = 0; stats->device_status = 0; stats->launches = 0; }
  if (len_hist) for (size_t z = 0; z < D; ++z) len_hist[z] = 0;
  cudaEvent_t t0 = e->ev[4], t1 = e->ev[5];
  int32_t* const table_dev = device_view(e, pinned, (size_t)n * D * 4);  // early delivery, where the table allows it
  cudaEventRecord(t0, streams[0]);
  bool pending[2] = {false, false};
  int batch_launches[2] = {0, 0};
  auto drain = [&](int s) -> int {
    if (!pending[s]) return FW_OK;
    FW_CUDA(cudaStreamSynchronize(streams[s]));
    float ms = 0.f;
    FW_CUDA(cudaEventElapsedTime(&ms, evs[s][0], evs[s][1]));
    pending[s] = false;
    return collect(hsc[s], p->d, ms, batch_launches[s], stats, len_hist, true);
  };
  int which = 0;
  fw_walk_params bp = *p;
  for (int64_t off = 0; off < n && !rc; off += batch_size, which ^= 1) {
    const int64_t m = std::min(batch_size, n - off);
    rc = drain(which);
    if (rc) break;
    cudaStream_t st = streams[which];
    bp.query_id_base = p->query_id_base + (uint64_t)off * (p->query_id_stride ? p->query_id_stride : 1);
    cudaError_t err = cudaMemcpyAsync(e->d_starts[which], starts_host + off, (size_t)m * 4, cudaMemcpyHostToDevice, st);
    if (err != cudaSuccess) { rc = fw::fail(FW_ERR_CUDA, "H2D copy failed: %s", cudaGetErrorString(err)); break; }
    bool delivered = false;
    rc = enqueue_walk(e, &bp, e->d_starts[which], m, e->d_result[which], st, evs[which][0], evs[which][1], dsc[which], hsc[which],
                      &batch_launches[which], table_dev ? table_dev + (size_t)off * D : nullptr, &delivered);
    if (rc) break;
    err = delivered ? cudaSuccess
                    : cudaMemcpyAsync(pinned + (size_t)off * D, e->d_result[which], (size_t)m * D * 4, cudaMemcpyDeviceToHost, st);
    if (err != cudaSuccess) { rc = fw::fail(FW_ERR_CUDA, "D2H copy failed: %s", cudaGetErrorString(err)); break; }
    pending[which] = true;
  }
  if (!rc) rc = drain(0);
  if (!rc) rc = drain(1);
  if (!rc) {
    cudaEventRecord(t1, streams[0]);
    cudaEventSynchronize(t1);
    float total = 0.f;
    cudaEventElapsedTime(&total, t0, t1);
    if (stats) stats->total_ms = total;
  }
  if (rc) return bail(rc);
  return FW_OK;
}

// walk_batch (include/walker.cuh:54-57, src/walk.cu:576-649): the callee allocates the pinned result.
extern "C" int fw_walk_batch(fw_engine* e, const fw_walk_params* p, const int32_t* starts_host,
                             int64_t n, int64_t batch_size, int32_t headroom_mb,
                             int32_t** result_pinned, fw_walk_stats* stats, uint64_t* len_hist) {
  fw::clear_error();
  int rc = check_params(e, p, n);
  if (rc) return rc;
  if (!result_pinned || (n > 0 && !starts_host)) return fw::fail(FW_ERR_ARG, "null buffer");
  *result_pinned = nullptr;
  DeviceGuard guard(e->device);
  int32_t* pinned = nullptr;
  cudaError_t err = cudaMallocHost(&pinned, std::max<size_t>((size_t)n * ((size_t)p->d + 1) * 4, 4));
  if (err != cudaSuccess) return fw::fail(FW_ERR_NOMEM, "cudaMallocHost failed: %s", cudaGetErrorString(err));
  rc = walk_batches(e, p, starts_host, n, batch_size, headroom_mb, pinned, stats, len_hist);
  if (rc) { cudaFreeHost(pinned); return rc; }
  *result_pinned = pinned;
  return FW_OK;
}

// Same pipeline into a buffer the caller owns (page-locked memory lets the copies overlap the walks).
extern "C" int fw_walk_batch_into(fw_engine* e, const fw_walk_params* p, const int32_t* starts_host,
                                  int64_t n, int64_t batch_size, int32_t headroom_mb,
                                  int32_t* result_host, fw_walk_stats* stats, uint64_t* len_hist) {
  fw::clear_error();
  int rc = check_params(e, p, n);
  if (rc) return rc;
  if (n > 0 && (!starts_host || !result_host)) return fw::fail(FW_ERR_ARG, "null buffer");
  return walk_batches(e, p, starts_host, n, batch_size, headroom_mb, result_host, stats, len_hist);
}

// ---------------------------------------------------------------------------
// Self-test of the bounded wait
// ---------------------------------------------------------------------------
namespace {
// One warp waits on an mbarrier that nothing ever arrives at, with the same polling loop the
// ring uses but a caller-chosen limit; it must come back and report, not spin.
__global__ void wait_timeout_probe(uint32_t polls, unsigned int* out) {
  __shared__ __align__(8) unsigned long long bar;
  const uint32_t addr = smem_addr(&bar);
  if (threadIdx.x == 0) {
    mbar_init(addr, 1u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  bool done = false;
  for (uint32_t i = 0; i < polls && !done; ++i) done = mbar_try_wait(addr, 0u) != 0;
  if (!done && threadIdx.x == 0) atomicOr(out, FW_STATUS_WAIT_TIMEOUT);
}
}  // namespace

extern "C" int fw_selftest_wait_timeout(int device, uint32_t polls, uint32_t* status) {
  fw::clear_error();
  if (!status) return fw::fail(FW_ERR_ARG, "fw_selftest_wait_timeout: null argument");
  if (polls == 0 || polls > (1u << 20)) return fw::fail(FW_ERR_ARG, "polls must be in 1..2^20");
  DeviceGuard guard(device);
  if (!guard.ok) return fw::fail(FW_ERR_ARG, "device %d cannot be made current", device);
  unsigned int* d = nullptr;
  FW_CUDA(cudaMalloc(&d, sizeof(unsigned int)));
  cudaError_t err = cudaMemset(d, 0, sizeof(unsigned int));
  if (err == cudaSuccess) { wait_timeout_probe<<<1, 32>>>(polls, d); err = cudaGetLastError(); }
  unsigned int h = 0;
  if (err == cudaSuccess) err = cudaMemcpy(&h, d, sizeof(h), cudaMemcpyDeviceToHost);
  cudaFree(d);
  if (err != cudaSuccess) return fw::fail(FW_ERR_CUDA, "wait self-test failed: %s", cudaGetErrorString(err));
  *status = h;
  return FW_OK;
}

// ---------------------------------------------------------------------------
// Allocation-free entry point
// ---------------------------------------------------------------------------
//
// Some hosts of this library may not allocate device memory at call time: a
// plugin running inside another framework's memory pool that has already
// reserved the whole GPU, a latency-critical serving loop where a cudaMalloc
// would serialise the device, or code running after start-up in a process
// whose allocator has been frozen.  For them the walk's scratch (the query
// counter, the step/scanned/status counters and the walk-length histogram)
// lives in a fixed array that is part of the loaded module.  Every GPU that
// loads the library holds these 32 KB + 32 B until the process exits.
namespace {
constexpr int kNoAllocMaxD = 4095;  // largest `d` the fixed scratch can serve
constexpr int kNoAllocWords = kSlotHist + kNoAllocMaxD + 1;
constexpr int kNoAllocMaxDevices = 64;
}  // namespace

static __device__ __align__(256) unsigned long long g_noalloc_scratch[kNoAllocWords];

namespace {
// Device address of g_noalloc_scratch per device ordinal.  In host code the
// array's name is only a handle for the runtime, so the address each kernel
// receives is looked up once per device, with that device current.
unsigned long long* g_noalloc_ptr[kNoAllocMaxDevices] = {};

int noalloc_scratch_for(int device, unsigned long long** out) {
  if (device < 0 || device >= kNoAllocMaxDevices)
    return fw::fail(FW_ERR_ARG, "device ordinal %d is beyond the %d this entry point supports", device,
                    kNoAllocMaxDevices);
  static std::mutex table_mu;
  std::lock_guard<std::mutex> lock(table_mu);
  if (!g_noalloc_ptr[device]) {
    int now = -1;
    if (cudaGetDevice(&now) != cudaSuccess || now != device)
      return fw::fail(FW_ERR_CUDA, "device %d is not current; the scratch address cannot be looked up", device);
    void* p = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (err != cudaSuccess || !p)
      return fw::fail(FW_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed on device %d: %s", device,
                      cudaGetErrorString(err));
    g_noalloc_ptr[device] = static_cast<unsigned long long*>(p);
  }
  *out = g_noalloc_ptr[device];
  return FW_OK;
}
}  // namespace

extern "C" int fw_walk_csr_noalloc(int device, int64_t V, int64_t E, const void* xadj_dev, int xadj_bits,
                                   const int32_t* adj_dev, const float* weight_dev,
                                   const int32_t* label_dev, const fw_walk_params* p,
                                   const int32_t* starts_dev, int64_t n, int32_t* result_dev,
                                   void* stream, fw_walk_stats* stats, uint64_t* len_hist) {
  fw::clear_error();
  if (!p) return fw::fail(FW_ERR_ARG, "null params");
  if (V < 0 || E < 0 || n < 0 || !xadj_dev || !adj_dev) return fw::fail(FW_ERR_ARG, "bad sizes or null CSR arrays");
  if (xadj_bits != 32 && xadj_bits != 64) return fw::fail(FW_ERR_ARG, "xadj_bits must be 32 or 64");
  if (p->app < FW_APP_DEEPWALK || p->app > FW_APP_METAPATH) return fw::fail(FW_ERR_ARG, "unknown app %d", p->app);
  if (p->d < 0 || p->d > kNoAllocMaxD)
    return fw::fail(FW_ERR_ARG, "d=%d exceeds the fixed scratch of this entry point (max %d); use fw_walk_device",
                    p->d, kNoAllocMaxD);
  if (p->group_mode != 0 && p->group_mode != FW_GROUP_EDGE && p->group_mode != FW_GROUP_STRIP)
    return fw::fail(FW_ERR_ARG, "group_mode must be 0, %d or %d", FW_GROUP_EDGE, FW_GROUP_STRIP);
  if (p->app == FW_APP_METAPATH) {
    if (!label_dev) return fw::fail(FW_ERR_ARG, "MetaPath needs edge labels");
    if (!p->schema || p->schema_len <= 0 || p->schema_len > kMaxSchema)
      return fw::fail(FW_ERR_ARG, "schema length must be in 1..%d", kMaxSchema);
  } else if (!weight_dev) {
    return fw::fail(FW_ERR_ARG, "this app needs edge weights");
  }
  if (p->app == FW_APP_NODE2VEC && !(p->p > 0.0 && p->q > 0.0)) return fw::fail(FW_ERR_ARG, "node2vec needs p > 0 and q > 0");
  if (n > 0 && (!starts_dev || !result_dev)) return fw::fail(FW_ERR_ARG, "null device buffer");
  if (((uintptr_t)adj_dev | (uintptr_t)weight_dev | (uintptr_t)label_dev) & 15u)
    return fw::fail(FW_ERR_ARG, "edge arrays must be 16-byte aligned");
  int count = 0, cc_major = 0;
  FW_CUDA(cudaGetDeviceCount(&count));
  if (device < 0 || device >= count) return fw::fail(FW_ERR_ARG, "device %d out of range (%d visible)", device, count);
  FW_CUDA(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, device));
  if (cc_major < 10) return fw::fail(FW_ERR_CUDA, "device %d is below sm_100; this library is built for sm_100a only", device);
  DeviceGuard guard(device);
  if (!guard.ok) return fw::fail(FW_ERR_CUDA, "cudaSetDevice(%d) failed", device);
  unsigned long long* scratch = nullptr;
  int rc = noalloc_scratch_for(device, &scratch);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  WalkArgs a;
  a.xadj = xadj_dev; a.adj = adj_dev; a.weight = weight_dev; a.label = label_dev;
  a.V = V; a.starts = starts_dev; a.n = n; a.result = result_dev; a.scratch = scratch;
  a.qid_base = p->query_id_base; a.qid_stride = p->query_id_stride ? p->query_id_stride : 1; a.d = p->d;
  a.tp_thresh = fw::tp_threshold(p->tp);
  a.inv_p = (float)(1.0 / p->p); a.inv_q = (float)(1.0 / p->q);
  a.n2v_fmax = std::max(1.0f, std::max(a.inv_p, a.inv_q)) * 1.00001f;
  a.k0 = (uint32_t)p->seed; a.k1 = (uint32_t)(p->seed >> 32);
  fw::philox_round_keys(a.k0, a.k1, a.rk);
  a.hist_in_smem = 1;  // d + 1 <= 4096 words always fits
  a.schema_len = p->app == FW_APP_METAPATH ? p->schema_len : 1;
  for (int i = 0; i < kMaxSchema; ++i)
    a.schema[i] = (p->app == FW_APP_METAPATH && i < p->schema_len) ? p->schema[i] : 0;
  const int mode = p->group_mode == 0 ? FW_GROUP_STRIP : p->group_mode;
  KernelFn fn = pick_kernel(p->app, mode, /*clean=*/false, /*shared=*/false, xadj_bits);  // caller's arrays: not inspected
  const size_t smem = kernel_smem_bytes(p->app, mode, p->d, true);
  int per_sm = 0, sms = 0;
  rc = prepare_kernel(fn, smem, &per_sm);
  if (rc) return rc;
  FW_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  const size_t words = (size_t)kSlotHist + (size_t)p->d + 1;
  // the array keeps the previous call's counters: everything this call reads starts at zero
  FW_CUDA(cudaMemsetAsync(scratch, 0, words * 8, st));
  if (n > 0) {
    const int64_t want = (n + (kThreads / 32) * kMinClaim - 1) / ((kThreads / 32) * kMinClaim);
    const int grid = (int)std::min<int64_t>((int64_t)sms * per_sm, std::max<int64_t>(want, 1));
    void* params[] = {&a};
    FW_CUDA(cudaLaunchKernel((const void*)fn, dim3(grid), dim3(kThreads), params, smem, st));
  }
  // counters go straight into the caller's memory, in two plain copies
  unsigned long long head[kSlotHist];
  FW_CUDA(cudaMemcpyAsync(head, scratch, sizeof(head), cudaMemcpyDeviceToHost, st));
  if (len_hist)
    FW_CUDA(cudaMemcpyAsync(len_hist, scratch + kSlotHist, (size_t)(p->d + 1) * 8, cudaMemcpyDeviceToHost, st));
  FW_CUDA(cudaStreamSynchronize(st));
  if (stats) {
    stats->steps = head[kSlotSteps];
    stats->scanned = head[kSlotScanned];
    stats->device_status = (uint32_t)head[kSlotStatus];
    stats->device_ms = 0.0;
    stats->total_ms = 0.0;
    stats->launches = n > 0 ? 1 : 0;
  }
  if (head[kSlotStatus] & FW_STATUS_WAIT_TIMEOUT)
    return fw::fail(FW_ERR_DEVICE, "the walk kernel gave up waiting for a staged copy; the result is incomplete");
  return FW_OK;
}

#ifdef FW_PHASE_TIMERS
// Development aid (only in builds with -DFW_PHASE_TIMERS): reads, and optionally clears, the
// per-phase cycle counters of the current device.
extern "C" int fw_debug_profile(unsigned long long* out16, int reset) {
  if (out16 && cudaMemcpyFromSymbol(out16, g_prof, sizeof(unsigned long long) * 16) != cudaSuccess)
    return fw::fail(FW_ERR_CUDA, "cudaMemcpyFromSymbol failed");
  if (reset) {
    unsigned long long zero[16] = {};
    if (cudaMemcpyToSymbol(g_prof, zero, sizeof(zero)) != cudaSuccess) return fw::fail(FW_ERR_CUDA, "cudaMemcpyToSymbol failed");
  }
  return FW_OK;
}
#endif
