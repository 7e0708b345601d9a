// Host CSR container and the on-disk format.
//
// File layout (little endian, no padding), as read by the reference loader
// (include/graph.cuh:93-190) and written by its converter
// (data/EdgeListToCSR.cpp:217-251):
//   <prefix>_xadj.bin   int32 V, uint32 E, then uint32 xadj[V+1]
//   <prefix>_edge.bin   int32 adj[E]
//   <prefix>_weight.bin float32 w[E]
//   <prefix>_label.bin  int32 label[E]
// Extension for graphs with E >= 2^32: the same 8-byte header (E saturated to
// 0xFFFFFFFF when it does not fit) followed by int64 xadj[V+1]; told apart by
// the file size.
#include <errno.h>
#include <math.h>
#include <stdio.h>
#include <string.h>
#include <sys/stat.h>

#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>

#include "fw_internal.h"
#include "fw_spec.cuh"

namespace fw {
static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
void clear_error() { g_err[0] = 0; }
}  // namespace fw

extern "C" const char* fw_last_error(void) { return fw::g_err; }

namespace {

int64_t file_size(const std::string& path) {
  struct stat st;
  if (stat(path.c_str(), &st) != 0) return -1;
  return (int64_t)st.st_size;
}

// Reads `bytes` bytes at `offset` into a fresh malloc buffer.
int read_block(const std::string& path, int64_t offset, int64_t bytes, void** out) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return fw::fail(FW_ERR_IO, "cannot open %s: %s", path.c_str(), strerror(errno));
  void* buf = malloc(bytes > 0 ? (size_t)bytes : 1);
  if (!buf) { fclose(f); return fw::fail(FW_ERR_NOMEM, "out of host memory (%lld bytes)", (long long)bytes); }
  if (fseeko(f, offset, SEEK_SET) != 0 ||
      (bytes > 0 && fread(buf, 1, (size_t)bytes, f) != (size_t)bytes)) {
    fclose(f); free(buf);
    return fw::fail(FW_ERR_IO, "short read from %s", path.c_str());
  }
  fclose(f);
  *out = buf;
  return FW_OK;
}

int write_block(FILE* f, const void* p, int64_t bytes, const std::string& path) {
  if (bytes > 0 && fwrite(p, 1, (size_t)bytes, f) != (size_t)bytes)
    return fw::fail(FW_ERR_IO, "short write to %s", path.c_str());
  return FW_OK;
}

int validate(const fw_graph* g) {
  if (fw::row_begin(g, 0) != 0) return fw::fail(FW_ERR_IO, "xadj[0] is not 0");
  int64_t prev = 0;
  for (int64_t v = 1; v <= g->V; ++v) {
    const int64_t x = fw::row_begin(g, v);
    if (x < prev) return fw::fail(FW_ERR_IO, "xadj decreases at vertex %lld", (long long)v);
    prev = x;
  }
  if (prev != g->E)
    return fw::fail(FW_ERR_IO, "xadj[V]=%lld does not match the edge count %lld",
                    (long long)prev, (long long)g->E);
  return FW_OK;
}

}  // namespace

extern "C" void fw_graph_destroy(fw_graph* g) {
  if (!g) return;
  free(g->xadj); free(g->adj); free(g->weight); free(g->label);
  delete g;
}

extern "C" int fw_graph_load(const char* prefix, int need_weight, int need_label, fw_graph** out) {
  fw::clear_error();
  if (!prefix || !out) return fw::fail(FW_ERR_ARG, "fw_graph_load: null argument");
  *out = nullptr;
  const std::string p(prefix);
  const std::string fx = p + "_xadj.bin", fe = p + "_edge.bin";
  const int64_t sx = file_size(fx), se = file_size(fe);
  if (sx < 0) return fw::fail(FW_ERR_IO, "cannot open %s", fx.c_str());
  if (se < 0) return fw::fail(FW_ERR_IO, "cannot open %s", fe.c_str());
  if (sx < 8 + 4) return fw::fail(FW_ERR_IO, "%s is too short for a header", fx.c_str());
  void* hdr = nullptr;
  int rc = read_block(fx, 0, 8, &hdr);
  if (rc) return rc;
  int32_t V32; uint32_t E32;
  memcpy(&V32, hdr, 4); memcpy(&E32, (char*)hdr + 4, 4);
  free(hdr);
  if (V32 < 0) return fw::fail(FW_ERR_IO, "%s: negative vertex count", fx.c_str());
  fw_graph* g = new fw_graph();
  g->V = V32;
  if (sx == 8 + 4 * (g->V + 1)) g->xadj_bits = 32;
  else if (sx == 8 + 8 * (g->V + 1)) g->xadj_bits = 64;
  else {
    delete g;
    return fw::fail(FW_ERR_IO, "%s: size %lld matches neither 32- nor 64-bit offsets for V=%d",
                    fx.c_str(), (long long)sx, V32);
  }
  if (se % 4 != 0) { delete g; return fw::fail(FW_ERR_IO, "%s: size is not a multiple of 4", fe.c_str()); }
  g->E = se / 4;
  if (g->xadj_bits == 32 && (int64_t)E32 != g->E) {
    delete g;
    return fw::fail(FW_ERR_IO, "%s: header says %u edges, %s holds %lld", fx.c_str(), E32,
                    fe.c_str(), (long long)(se / 4));
  }
  rc = read_block(fx, 8, (g->xadj_bits / 8) * (g->V + 1), &g->xadj);
  if (!rc) rc = read_block(fe, 0, se, (void**)&g->adj);
  if (!rc) rc = validate(g);
  if (!rc && need_weight) {
    const std::string fwt = p + "_weight.bin";
    if (file_size(fwt) != 4 * g->E) rc = fw::fail(FW_ERR_IO, "%s: missing or wrong size", fwt.c_str());
    else rc = read_block(fwt, 0, 4 * g->E, (void**)&g->weight);
  }
  if (!rc && need_label) {
    const std::string fl = p + "_label.bin";
    if (file_size(fl) != 4 * g->E) rc = fw::fail(FW_ERR_IO, "%s: missing or wrong size", fl.c_str());
    else rc = read_block(fl, 0, 4 * g->E, (void**)&g->label);
  }
  if (rc) { fw_graph_destroy(g); return rc; }
  *out = g;
  return FW_OK;
}

extern "C" int fw_graph_save(const fw_graph* g, const char* prefix) {
  fw::clear_error();
  if (!g || !prefix) return fw::fail(FW_ERR_ARG, "fw_graph_save: null argument");
  if (g->V > INT32_MAX) return fw::fail(FW_ERR_ARG, "vertex count does not fit the int32 header");
  const std::string p(prefix);
  struct Part { std::string path; const void* data; int64_t bytes; };
  const Part parts[] = {
      {p + "_edge.bin", g->adj, 4 * g->E},
      {p + "_weight.bin", g->weight, g->weight ? 4 * g->E : -1},
      {p + "_label.bin", g->label, g->label ? 4 * g->E : -1},
  };
  {
    const std::string fx = p + "_xadj.bin";
    FILE* f = fopen(fx.c_str(), "wb");
    if (!f) return fw::fail(FW_ERR_IO, "cannot create %s: %s", fx.c_str(), strerror(errno));
    const int32_t V32 = (int32_t)g->V;
    const uint32_t E32 = g->E > 0xFFFFFFFFll ? 0xFFFFFFFFu : (uint32_t)g->E;
    int rc = write_block(f, &V32, 4, fx);
    if (!rc) rc = write_block(f, &E32, 4, fx);
    if (!rc) rc = write_block(f, g->xadj, (g->xadj_bits / 8) * (g->V + 1), fx);
    if (fclose(f) != 0 && !rc) rc = fw::fail(FW_ERR_IO, "cannot close %s", fx.c_str());
    if (rc) return rc;
  }
  for (const Part& part : parts) {
    if (part.bytes < 0) continue;
    FILE* f = fopen(part.path.c_str(), "wb");
    if (!f) return fw::fail(FW_ERR_IO, "cannot create %s: %s", part.path.c_str(), strerror(errno));
    int rc = write_block(f, part.data, part.bytes, part.path);
    if (fclose(f) != 0 && !rc) rc = fw::fail(FW_ERR_IO, "cannot close %s", part.path.c_str());
    if (rc) return rc;
  }
  return FW_OK;
}

extern "C" int fw_graph_from_arrays(int64_t V, int64_t E, const void* xadj, int xadj_bits,
                                    const int32_t* adj, const float* weight,
                                    const int32_t* label, fw_graph** out) {
  fw::clear_error();
  if (!out) return fw::fail(FW_ERR_ARG, "fw_graph_from_arrays: null output");
  *out = nullptr;
  if (V < 0 || E < 0 || !xadj || (E > 0 && !adj))
    return fw::fail(FW_ERR_ARG, "fw_graph_from_arrays: bad sizes or null arrays");
  if (V > INT32_MAX) return fw::fail(FW_ERR_ARG, "vertex ids are int32: V must be < 2^31");
  if (xadj_bits != 32 && xadj_bits != 64)
    return fw::fail(FW_ERR_ARG, "xadj_bits must be 32 or 64, got %d", xadj_bits);
  if (xadj_bits == 32 && E > 0xFFFFFFFFll)
    return fw::fail(FW_ERR_ARG, "E=%lld needs 64-bit offsets", (long long)E);
  fw_graph* g = new fw_graph();
  g->V = V; g->E = E; g->xadj_bits = xadj_bits;
  const size_t xb = (size_t)(xadj_bits / 8) * (size_t)(V + 1), eb = 4 * (size_t)E;
  g->xadj = malloc(xb);
  g->adj = (int32_t*)malloc(eb ? eb : 1);
  if (weight) g->weight = (float*)malloc(eb ? eb : 1);
  if (label) g->label = (int32_t*)malloc(eb ? eb : 1);
  if (!g->xadj || !g->adj || (weight && !g->weight) || (label && !g->label)) {
    fw_graph_destroy(g);
    return fw::fail(FW_ERR_NOMEM, "out of host memory");
  }
  memcpy(g->xadj, xadj, xb);
  if (eb) memcpy(g->adj, adj, eb);
  if (weight && eb) memcpy(g->weight, weight, eb);
  if (label && eb) memcpy(g->label, label, eb);
  const int rc = validate(g);
  if (rc) { fw_graph_destroy(g); return rc; }
  *out = g;
  return FW_OK;
}

extern "C" int fw_graph_info(const fw_graph* g, int64_t* V, int64_t* E, int32_t* xadj_bits,
                             int32_t* has_weight, int32_t* has_label) {
  if (!g) return fw::fail(FW_ERR_ARG, "fw_graph_info: null graph");
  if (V) *V = g->V;
  if (E) *E = g->E;
  if (xadj_bits) *xadj_bits = g->xadj_bits;
  if (has_weight) *has_weight = g->weight != nullptr;
  if (has_label) *has_label = g->label != nullptr;
  return FW_OK;
}

extern "C" int fw_graph_arrays(const fw_graph* g, const void** xadj, const int32_t** adj,
                               const float** weight, const int32_t** label) {
  if (!g) return fw::fail(FW_ERR_ARG, "fw_graph_arrays: null graph");
  if (xadj) *xadj = g->xadj;
  if (adj) *adj = g->adj;
  if (weight) *weight = g->weight;
  if (label) *label = g->label;
  return FW_OK;
}

extern "C" int fw_graph_max_degree(const fw_graph* g, int64_t* vertex, int64_t* degree) {
  if (!g) return fw::fail(FW_ERR_ARG, "fw_graph_max_degree: null graph");
  int64_t best = -1, arg = 0;
  for (int64_t v = 0; v < g->V; ++v) {
    const int64_t dg = fw::row_begin(g, v + 1) - fw::row_begin(g, v);
    if (dg > best) { best = dg; arg = v; }
  }
  if (vertex) *vertex = arg;
  if (degree) *degree = best < 0 ? 0 : best;
  return FW_OK;
}

// Edge list -> CSR with the conventions of the reference's converter (data/EdgeListToCSR.cpp:132-268):
// the graph is made undirected, duplicate edges are dropped, vertices are renumbered in order of
// first appearance (so vertices without an edge disappear), and every undirected edge gets one
// label and one weight shared by its two directions.  Differences, on purpose: rows come out
// sorted by neighbour id (node2vec's membership test needs that; the reference appends in input
// order), self-loops are dropped, and labels / weights are seeded (Philox keyed by the
// undirected edge's rank) instead of drawn from std::random_device.
extern "C" int fw_graph_from_edgelist(const char* path, int32_t n_labels, float weight_lo, float weight_hi,
                                      uint64_t seed, fw_graph** out) {
  fw::clear_error();
  if (!path || !out) return fw::fail(FW_ERR_ARG, "fw_graph_from_edgelist: null argument");
  *out = nullptr;
  FILE* f = fopen(path, "r");
  if (!f) return fw::fail(FW_ERR_IO, "cannot open %s: %s", path, strerror(errno));
  std::unordered_map<long long, int32_t> renum;
  std::vector<uint64_t> und;  // (min << 32 | max) of the renumbered endpoints
  char line[512];
  long long lineno = 0;
  while (fgets(line, sizeof(line), f)) {
    ++lineno;
    const char* p = line;
    while (*p == ' ' || *p == '\t') ++p;
    if (*p == '#' || *p == '%' || *p == '\n' || *p == '\r' || *p == 0) continue;
    long long u, v;
    if (sscanf(p, "%lld %lld", &u, &v) != 2) {
      fclose(f);
      return fw::fail(FW_ERR_IO, "%s:%lld: expected two vertex ids", path, lineno);
    }
    if (u == v) continue;
    int32_t ids[2];
    const long long raw[2] = {u, v};
    for (int k = 0; k < 2; ++k) {
      auto it = renum.find(raw[k]);
      if (it == renum.end()) {
        if (renum.size() >= (size_t)INT32_MAX) { fclose(f); return fw::fail(FW_ERR_ARG, "more than 2^31-1 vertices"); }
        it = renum.emplace(raw[k], (int32_t)renum.size()).first;
      }
      ids[k] = it->second;
    }
    const uint32_t lo = (uint32_t)std::min(ids[0], ids[1]), hi = (uint32_t)std::max(ids[0], ids[1]);
    und.push_back((uint64_t)lo << 32 | hi);
  }
  fclose(f);
  std::sort(und.begin(), und.end());
  und.erase(std::unique(und.begin(), und.end()), und.end());
  const int64_t V = (int64_t)renum.size(), E = 2 * (int64_t)und.size();
  if (E > 0xFFFFFFFFll) return fw::fail(FW_ERR_ARG, "more than 2^32-1 directed edges");
  struct Half { uint64_t key; uint32_t rank; };  // key = src << 32 | dst, rank = undirected edge
  std::vector<Half> half;
  half.reserve((size_t)E);
  for (size_t r = 0; r < und.size(); ++r) {
    const uint32_t lo = (uint32_t)(und[r] >> 32), hi = (uint32_t)und[r];
    half.push_back({(uint64_t)lo << 32 | hi, (uint32_t)r});
    half.push_back({(uint64_t)hi << 32 | lo, (uint32_t)r});
  }
  std::sort(half.begin(), half.end(), [](const Half& a, const Half& b) { return a.key < b.key; });
  fw_graph* g = new fw_graph();
  g->V = V; g->E = E; g->xadj_bits = 32;
  const bool weights = weight_hi > weight_lo, labels = n_labels > 0;
  g->xadj = malloc(4 * (size_t)(V + 1));
  g->adj = (int32_t*)malloc(E ? 4 * (size_t)E : 1);
  if (weights) g->weight = (float*)malloc(E ? 4 * (size_t)E : 1);
  if (labels) g->label = (int32_t*)malloc(E ? 4 * (size_t)E : 1);
  if (!g->xadj || !g->adj || (weights && !g->weight) || (labels && !g->label)) {
    fw_graph_destroy(g);
    return fw::fail(FW_ERR_NOMEM, "out of host memory");
  }
  uint32_t* xadj = (uint32_t*)g->xadj;
  int64_t e = 0;
  for (int64_t v = 0; v <= V; ++v) {
    while (e < E && (int64_t)(half[(size_t)e].key >> 32) < v) ++e;
    xadj[v] = (uint32_t)e;
  }
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (e = 0; e < E; ++e) {
    const Half& h = half[(size_t)e];
    g->adj[e] = (int32_t)(uint32_t)h.key;
    const fw::Philox4 r = fw::philox4x32_10(h.rank, 0u, 0u, 0x45u, k0, k1);
    if (weights) {
      const float w = fmaf((float)(r.x >> 8) * 0x1p-24f, weight_hi - weight_lo, weight_lo);
      g->weight[e] = w >= weight_hi ? weight_lo : w;
    }
    if (labels) g->label[e] = (int32_t)(((uint64_t)r.y * (uint32_t)n_labels) >> 32);
  }
  *out = g;
  return FW_OK;
}

// --lognorm (include/graph.cuh:79-91).  One Philox block per pair of values: words 0,1 -> u1 in
// (0,1), words 2,3 -> u2 in [0,1), each with 53 bits; Box-Muller gives z = r cos(t), r sin(t).
extern "C" int fw_lognormal_weights(int64_t n, double mean, double sigma, uint64_t seed, float* out) {
  fw::clear_error();
  if (n < 0 || (n > 0 && !out)) return fw::fail(FW_ERR_ARG, "fw_lognormal_weights: bad arguments");
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  const double two_pi = 6.283185307179586476925286766559;
  for (int64_t i = 0; i < n; i += 2) {
    const uint64_t blk = (uint64_t)i >> 1;
    const fw::Philox4 r = fw::philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), 0x4C4F474Eu, 0u, k0, k1);
    const uint64_t a = (((uint64_t)r.x << 32) | r.y) >> 11, b = (((uint64_t)r.z << 32) | r.w) >> 11;
    const double u1 = ((double)a + 0.5) * 0x1p-53, u2 = (double)b * 0x1p-53;
    const double rad = sqrt(-2.0 * log(u1)), ang = two_pi * u2;
    out[i] = (float)exp(mean + sigma * rad * cos(ang));
    if (i + 1 < n) out[i + 1] = (float)exp(mean + sigma * rad * sin(ang));
  }
  return FW_OK;
}
