// Seeded synthetic R-MAT graphs (Chakrabarti, Zhan, Faloutsos, SDM'04) in the
// engine's CSR form: directed, no self-loops, duplicate edges removed, rows
// sorted by neighbour id.  They stand in for the public graphs the reference
// downloads in data/get_dataset.sh, none of which ships with this code.
//
// Every edge and every attribute is a pure function of (seed, index) through
// Philox, so the host path and the device path produce identical graphs:
//   candidate i : level l of `scale` draws one 32-bit word, block counter
//                 (i_lo, i_hi, l>>2, 'R'), word l&3, compared with the integer
//                 thresholds of a, a+b, a+b+c;
//   weight[e]   : word e&3 of block (e>>2 lo, hi, 0, 'W') -> lo + (hi-lo)*u;
//   label[e]    : word e&3 of block (e>>2 lo, hi, 0, 'L') -> floor(u * n_labels).
#include <cuda_runtime.h>

#include <algorithm>
#include <cub/cub.cuh>
#include <unordered_set>
#include <vector>

#include "fw_internal.h"
#include "fw_spec.cuh"

namespace {

struct RmatCfg {
  int scale;
  uint32_t tA, tAB, tABC;
  uint32_t k0, k1;
  int64_t v_limit;  // 0 = none
};

uint32_t prob_threshold(double p) {
  const double t = p * 4294967296.0;
  if (!(t > 0)) return 0u;
  if (t >= 4294967295.0) return 0xFFFFFFFFu;
  return (uint32_t)t;
}

// Candidate edge i as (src << 32 | dst), or the sentinel 1 << (32+scale) when
// the candidate is a self-loop or touches an id >= v_limit.
FW_HD uint64_t rmat_candidate(const RmatCfg& c, uint64_t i) {
  uint32_t src = 0, dst = 0;
  fw::Philox4 r{0, 0, 0, 0};
  for (int l = 0; l < c.scale; ++l) {
    if ((l & 3) == 0)
      r = fw::philox4x32_10((uint32_t)i, (uint32_t)(i >> 32), (uint32_t)(l >> 2), 0x52u, c.k0, c.k1);
    const uint32_t x = (l & 3) == 0 ? r.x : (l & 3) == 1 ? r.y : (l & 3) == 2 ? r.z : r.w;
    const uint32_t sbit = x >= c.tAB ? 1u : 0u;
    const uint32_t dbit = (x >= c.tA && x < c.tAB) || x >= c.tABC ? 1u : 0u;
    src = (src << 1) | sbit;
    dst = (dst << 1) | dbit;
  }
  const bool bad = src == dst || (c.v_limit > 0 && ((int64_t)src >= c.v_limit || (int64_t)dst >= c.v_limit));
  return bad ? (1ull << (32 + c.scale)) : ((uint64_t)src << 32 | dst);
}

FW_HD uint32_t word_of(const fw::Philox4& r, uint32_t k) {
  return k == 0 ? r.x : k == 1 ? r.y : k == 2 ? r.z : r.w;
}

FW_HD float edge_weight(uint64_t e, float lo, float hi, uint32_t k0, uint32_t k1) {
  const uint64_t blk = e >> 2;
  const fw::Philox4 r = fw::philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), 0u, 0x57u, k0, k1);
  const float u = (float)(word_of(r, (uint32_t)e & 3u) >> 8) * 0x1p-24f;
  const float w = fmaf(u, hi - lo, lo);
  return w >= hi ? lo : w;
}

FW_HD int32_t edge_label(uint64_t e, uint32_t n_labels, uint32_t k0, uint32_t k1) {
  const uint64_t blk = e >> 2;
  const fw::Philox4 r = fw::philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), 0u, 0x4Cu, k0, k1);
  return (int32_t)(((uint64_t)word_of(r, (uint32_t)e & 3u) * n_labels) >> 32);
}

__global__ void k_candidates(RmatCfg c, int64_t n, uint64_t* keys) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    keys[i] = rmat_candidate(c, (uint64_t)i);
}

template <typename OffT>
__global__ void k_offsets(const uint64_t* keys, int64_t E, int64_t V, OffT* xadj) {
  for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v <= V;
       v += (int64_t)gridDim.x * blockDim.x) {
    const uint64_t target = (uint64_t)v << 32;
    int64_t lo = 0, hi = E;
    while (lo < hi) {
      const int64_t mid = lo + ((hi - lo) >> 1);
      if (keys[mid] < target) lo = mid + 1; else hi = mid;
    }
    xadj[v] = (OffT)lo;
  }
}

__global__ void k_attributes(const uint64_t* keys, int64_t E, int32_t* adj, float* weight,
                             float lo, float hi, uint32_t wk0, uint32_t wk1, int32_t* label,
                             uint32_t n_labels, uint32_t lk0, uint32_t lk1) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < E;
       e += (int64_t)gridDim.x * blockDim.x) {
    adj[e] = (int32_t)(uint32_t)keys[e];
    if (weight) weight[e] = edge_weight((uint64_t)e, lo, hi, wk0, wk1);
    if (label) label[e] = edge_label((uint64_t)e, n_labels, lk0, lk1);
  }
}

#define RM_CUDA(call)                                                              \
  do {                                                                             \
    cudaError_t err__ = (call);                                                    \
    if (err__ != cudaSuccess) {                                                    \
      rc = fw::fail(FW_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(err__)); \
      goto done;                                                                   \
    }                                                                              \
  } while (0)

int alloc_host(fw_graph* g, bool weights, bool labels) {
  const size_t eb = 4 * (size_t)g->E;
  g->xadj = malloc((size_t)(g->xadj_bits / 8) * (size_t)(g->V + 1));
  g->adj = (int32_t*)malloc(eb ? eb : 1);
  if (weights) g->weight = (float*)malloc(eb ? eb : 1);
  if (labels) g->label = (int32_t*)malloc(eb ? eb : 1);
  if (!g->xadj || !g->adj || (weights && !g->weight) || (labels && !g->label))
    return fw::fail(FW_ERR_NOMEM, "out of host memory for a graph of %lld edges", (long long)g->E);
  return FW_OK;
}

int generate_device(const fw_rmat_params* p, const RmatCfg& cfg, fw_graph* g) {
  int rc = FW_OK;
  int prev_dev = 0;
  uint64_t *keys = nullptr, *keys_alt = nullptr, *uniq = nullptr;
  int64_t* d_count = nullptr;
  void *tmp = nullptr, *d_xadj = nullptr;
  int32_t *d_adj = nullptr, *d_label = nullptr;
  float* d_weight = nullptr;
  size_t tmp_bytes = 0, tmp2 = 0;
  const int64_t n = p->draws;
  const bool weights = p->weight_hi > p->weight_lo, labels = p->n_labels > 0;
  int64_t E = 0;
  const int threads = 256, blocks = 148 * 8;
  cudaGetDevice(&prev_dev);
  RM_CUDA(cudaSetDevice(p->device));
  RM_CUDA(cudaMalloc(&keys, 8 * (size_t)n));
  RM_CUDA(cudaMalloc(&keys_alt, 8 * (size_t)n));
  RM_CUDA(cudaMalloc(&d_count, 8));
  k_candidates<<<blocks, threads>>>(cfg, n, keys);
  RM_CUDA(cudaGetLastError());
  {
    cub::DoubleBuffer<uint64_t> db(keys, keys_alt);
    RM_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, tmp_bytes, db, n, 0, 33 + cfg.scale));
    RM_CUDA(cub::DeviceSelect::Unique(nullptr, tmp2, keys, keys_alt, d_count, n));
    tmp_bytes = std::max(tmp_bytes, tmp2);
    RM_CUDA(cudaMalloc(&tmp, tmp_bytes));
    RM_CUDA(cub::DeviceRadixSort::SortKeys(tmp, tmp_bytes, db, n, 0, 33 + cfg.scale));
    uint64_t* sorted = db.Current();
    uniq = db.Alternate();
    RM_CUDA(cub::DeviceSelect::Unique(tmp, tmp_bytes, sorted, uniq, d_count, n));
  }
  RM_CUDA(cudaMemcpy(&E, d_count, 8, cudaMemcpyDeviceToHost));
  if (E > 0) {  // the sentinel, if any candidate was dropped, sorts last
    uint64_t last = 0;
    RM_CUDA(cudaMemcpy(&last, uniq + (E - 1), 8, cudaMemcpyDeviceToHost));
    if (last == (1ull << (32 + cfg.scale))) --E;
  }
  g->E = E;
  if (g->xadj_bits == 32 && E > 0xFFFFFFFFll) {
    rc = fw::fail(FW_ERR_ARG, "%lld edges need xadj_bits = 64", (long long)E);
    goto done;
  }
  RM_CUDA(cudaMalloc(&d_xadj, (size_t)(g->xadj_bits / 8) * (size_t)(g->V + 1)));
  RM_CUDA(cudaMalloc(&d_adj, 4 * (size_t)std::max<int64_t>(E, 1)));
  if (weights) RM_CUDA(cudaMalloc(&d_weight, 4 * (size_t)std::max<int64_t>(E, 1)));
  if (labels) RM_CUDA(cudaMalloc(&d_label, 4 * (size_t)std::max<int64_t>(E, 1)));
  if (g->xadj_bits == 64) k_offsets<int64_t><<<blocks, threads>>>(uniq, E, g->V, (int64_t*)d_xadj);
  else k_offsets<uint32_t><<<blocks, threads>>>(uniq, E, g->V, (uint32_t*)d_xadj);
  k_attributes<<<blocks, threads>>>(uniq, E, d_adj, d_weight, p->weight_lo, p->weight_hi,
                                    (uint32_t)p->weight_seed, (uint32_t)(p->weight_seed >> 32),
                                    d_label, (uint32_t)p->n_labels, (uint32_t)p->label_seed,
                                    (uint32_t)(p->label_seed >> 32));
  RM_CUDA(cudaGetLastError());
  rc = alloc_host(g, weights, labels);
  if (rc) goto done;
  RM_CUDA(cudaMemcpy(g->xadj, d_xadj, (size_t)(g->xadj_bits / 8) * (size_t)(g->V + 1), cudaMemcpyDeviceToHost));
  RM_CUDA(cudaMemcpy(g->adj, d_adj, 4 * (size_t)E, cudaMemcpyDeviceToHost));
  if (weights) RM_CUDA(cudaMemcpy(g->weight, d_weight, 4 * (size_t)E, cudaMemcpyDeviceToHost));
  if (labels) RM_CUDA(cudaMemcpy(g->label, d_label, 4 * (size_t)E, cudaMemcpyDeviceToHost));
done:
  cudaFree(keys); cudaFree(keys_alt); cudaFree(d_count); cudaFree(tmp);
  cudaFree(d_xadj); cudaFree(d_adj); cudaFree(d_weight); cudaFree(d_label);
  cudaSetDevice(prev_dev);
  return rc;
}

int generate_host(const fw_rmat_params* p, const RmatCfg& cfg, fw_graph* g) {
  const uint64_t sentinel = 1ull << (32 + cfg.scale);
  std::vector<uint64_t> keys;
  if (p->e_target > 0) {
    // shortest prefix of the candidate stream holding e_target distinct edges
    std::unordered_set<uint64_t> seen;
    seen.reserve((size_t)p->e_target * 2);
    const uint64_t limit = (uint64_t)p->e_target * 1024u + 1024u;
    uint64_t i = 0;
    for (; (int64_t)seen.size() < p->e_target && i < limit; ++i) {
      const uint64_t k = rmat_candidate(cfg, i);
      if (k != sentinel) seen.insert(k);
    }
    if ((int64_t)seen.size() < p->e_target)
      return fw::fail(FW_ERR_ARG, "could not reach %lld distinct edges", (long long)p->e_target);
    keys.assign(seen.begin(), seen.end());
  } else {
    keys.reserve((size_t)p->draws);
    for (int64_t i = 0; i < p->draws; ++i) {
      const uint64_t k = rmat_candidate(cfg, (uint64_t)i);
      if (k != sentinel) keys.push_back(k);
    }
  }
  std::sort(keys.begin(), keys.end());
  keys.erase(std::unique(keys.begin(), keys.end()), keys.end());
  g->E = (int64_t)keys.size();
  if (g->xadj_bits == 32 && g->E > 0xFFFFFFFFll)
    return fw::fail(FW_ERR_ARG, "%lld edges need xadj_bits = 64", (long long)g->E);
  const bool weights = p->weight_hi > p->weight_lo, labels = p->n_labels > 0;
  const int rc = alloc_host(g, weights, labels);
  if (rc) return rc;
  int64_t e = 0;
  for (int64_t v = 0; v <= g->V; ++v) {
    while (e < g->E && (int64_t)(keys[(size_t)e] >> 32) < v) ++e;
    if (g->xadj_bits == 64) ((int64_t*)g->xadj)[v] = e; else ((uint32_t*)g->xadj)[v] = (uint32_t)e;
  }
  for (e = 0; e < g->E; ++e) {
    g->adj[e] = (int32_t)(uint32_t)keys[(size_t)e];
    if (weights)
      g->weight[e] = edge_weight((uint64_t)e, p->weight_lo, p->weight_hi, (uint32_t)p->weight_seed,
                                 (uint32_t)(p->weight_seed >> 32));
    if (labels)
      g->label[e] = edge_label((uint64_t)e, (uint32_t)p->n_labels, (uint32_t)p->label_seed,
                               (uint32_t)(p->label_seed >> 32));
  }
  return FW_OK;
}

}  // namespace

extern "C" int fw_rmat_generate(const fw_rmat_params* p, fw_graph** out) {
  fw::clear_error();
  if (!p || !out) return fw::fail(FW_ERR_ARG, "fw_rmat_generate: null argument");
  *out = nullptr;
  if (p->scale < 1 || p->scale > 30) return fw::fail(FW_ERR_ARG, "scale must be in 1..30");
  if (p->xadj_bits != 32 && p->xadj_bits != 64) return fw::fail(FW_ERR_ARG, "xadj_bits must be 32 or 64");
  if (p->draws < 0 || (p->draws == 0 && p->e_target <= 0)) return fw::fail(FW_ERR_ARG, "nothing to draw");
  if (!(p->a >= 0 && p->b >= 0 && p->c >= 0 && p->a + p->b + p->c <= 1.0 + 1e-12))
    return fw::fail(FW_ERR_ARG, "a, b, c must be probabilities with a+b+c <= 1");
  if (p->v_limit > (1ll << p->scale)) return fw::fail(FW_ERR_ARG, "v_limit exceeds 2^scale");
  if (p->e_target > 0 && p->device >= 0)
    return fw::fail(FW_ERR_ARG, "e_target is a host-only mode (device must be -1)");
  RmatCfg cfg;
  cfg.scale = p->scale;
  cfg.tA = prob_threshold(p->a);
  cfg.tAB = prob_threshold(p->a + p->b);
  cfg.tABC = prob_threshold(p->a + p->b + p->c);
  cfg.k0 = (uint32_t)p->seed;
  cfg.k1 = (uint32_t)(p->seed >> 32);
  cfg.v_limit = p->v_limit > 0 ? p->v_limit : 0;
  fw_graph* g = new fw_graph();
  g->V = p->v_limit > 0 ? p->v_limit : (1ll << p->scale);
  g->xadj_bits = p->xadj_bits;
  const int rc = p->device >= 0 ? generate_device(p, cfg, g) : generate_host(p, cfg, g);
  if (rc) { fw_graph_destroy(g); return rc; }
  *out = g;
  return FW_OK;
}
