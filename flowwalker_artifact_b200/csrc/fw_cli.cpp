// flowwalker: command-line front end with the reference's flags (src/main.cu:40-80), its flag
// rewriting (src/main.cu:244-272), start points (src/main.cu:273-296) and result consumers
// (src/main.cu:82-224), on top of the C ABI of libflowwalker.  Host C++ only.
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <map>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "../../include/flowwalker.h"
#include "fw_flags.h"

namespace {

using fwflags::Flag;

void define_flags(fwflags::Parser& fl) {
  fl.add("input", Flag::kString, "../data/wiki-Vote", "input dataset prefix");
  fl.add("b_file", Flag::kString, "../res/bucket.csv", "degree bucket file");
  fl.add("n", Flag::kInt, "4000", "sample size");
  fl.add("seq", Flag::kBool, "false", "start from 0 to n-1");
  fl.add("all", Flag::kBool, "false", "start from all nodes");
  fl.add("d", Flag::kInt, "80", "depth");
  fl.add("umgraph", Flag::kBool, "false", "edge arrays in unified memory (graphs larger than device memory)");
  fl.add("deepwalk", Flag::kBool, "false", "deepwalk");
  fl.add("node2vec", Flag::kBool, "false", "node2vec");
  fl.add("ppr", Flag::kBool, "false", "ppr");
  fl.add("metapath", Flag::kBool, "false", "metapath");
  fl.add("dprs", Flag::kBool, "false", "accepted for compatibility (one sampler serves every app)");
  fl.add("p", Flag::kDouble, "2.0", "hyper-parameter p for node2vec");
  fl.add("q", Flag::kDouble, "0.5", "hyper-parameter q for node2vec");
  fl.add("tp", Flag::kDouble, "0.2", "terminate probability");
  fl.add("schemalen", Flag::kInt, "5", "number of labels");
  fl.add("schema", Flag::kString, "0,1,2,3,4", "metapath schema");
  fl.add("printresult", Flag::kBool, "false", "print the first 100 walks (all walks with edge labels for metapath)");
  fl.add("printworkload", Flag::kBool, "false", "print sampled vertices / scanned edges");
  fl.add("save_degree", Flag::kBool, "false", "save the degree histogram of visited vertices to --b_file");
  fl.add("autobatch", Flag::kBool, "false", "use adaptive batch size");
  fl.add("batch", Flag::kBool, "false", "use batch mode");
  fl.add("syn", Flag::kBool, "false", "accepted for compatibility (batches are always double-buffered)");
  fl.add("batchsize", Flag::kInt, "10000000", "batch size");
  fl.add("headroom", Flag::kInt, "512", "GPU memory headroom while using autobatch (MB)");
  fl.add("walkmode", Flag::kInt, "-1", "accepted for compatibility (the reference's ablation kernels do not exist here)");
  fl.add("lognorm", Flag::kBool, "false", "replace the edge weights by seeded log-normal(0,3) weights");
  // additions
  fl.add("seed", Flag::kInt, "1337", "walk seed (Philox key)");
  fl.add("startseed", Flag::kInt, "4", "seed of the random start points (the reference uses time(NULL))");
  fl.add("uniformstarts", Flag::kBool, "false", "ppr: seeded uniform start points instead of the max-degree vertex");
  fl.add("group", Flag::kInt, "0", "sampler granularity: 0 default, 1 per neighbour, 64 per strip");
  fl.add("gpus", Flag::kInt, "1", "number of GPUs: queries are sharded, the graph is replicated");
  fl.add("shards", Flag::kInt, "0", "query shards (0 = one per GPU); shard r walks ids [r*n/S, (r+1)*n/S) on GPU r mod --gpus with a replica of its own");
  fl.add("interleave", Flag::kBool, "false", "shard r of S walks the ids r, r+S, r+2S, ... instead of a contiguous id range");
  fl.add("save_result", Flag::kString, "", "write the int32 [n x (d+1)] walk table to this file");
  fl.add("edgelist", Flag::kString, "", "build the graph from this text edge list instead of reading --input");
  fl.add("save_csr", Flag::kString, "", "write the graph as <prefix>_xadj/_edge/_weight/_label.bin and exit");
}

bool parse_schema(const std::string& text, std::vector<int32_t>* out) {
  size_t pos = 0;
  while (pos <= text.size()) {
    size_t comma = text.find(',', pos);
    if (comma == std::string::npos) comma = text.size();
    const std::string tok = text.substr(pos, comma - pos);
    char* end = nullptr;
    const long v = strtol(tok.c_str(), &end, 10);
    if (tok.empty() || !end || *end) return false;
    out->push_back((int32_t)v);
    pos = comma + 1;
  }
  return !out->empty();
}

int64_t row_begin(const void* xadj, int bits, int64_t v) {
  return bits == 64 ? static_cast<const int64_t*>(xadj)[v] : (int64_t) static_cast<const uint32_t*>(xadj)[v];
}

struct GraphView {
  int64_t V = 0, E = 0;
  int32_t bits = 32;
  const void* xadj = nullptr;
  const int32_t* adj = nullptr;
  const float* weight = nullptr;
  const int32_t* label = nullptr;
  int64_t degree(int64_t v) const { return row_begin(xadj, bits, v + 1) - row_begin(xadj, bits, v); }
};

// src/main.cu:151-181
void print_res(int64_t n, int depth, const int32_t* result) {
  unsigned long long sampled = 0;
  for (int64_t i = 0; i < 100 && i < n; ++i) {
    printf("----------------------\nWalker %lld:\n", (long long)i);
    int len = depth;
    for (int j = 0; j < depth; ++j) {
      const int32_t v = result[i * depth + j];
      if (v == -1) { len = j; break; }
      if (j > 0) ++sampled;
      printf("%d\t", v);
    }
    printf("\nTotal length=%d\n", len);
  }
  printf("Total sampled: %llu\n", sampled);
}

// src/main.cu:183-224
void print_res_metapath(int64_t n, int depth, const int32_t* result, const GraphView& g) {
  unsigned long long sampled = 0;
  for (int64_t i = 0; i < n; ++i) {
    printf("----------------------\nWalker %lld:\n", (long long)i);
    int len = depth;
    int32_t pre = -1;
    for (int j = 0; j < depth; ++j) {
      const int32_t v = result[i * depth + j];
      if (v == -1) { len = j; break; }
      if (pre != -1) {
        const int64_t b = row_begin(g.xadj, g.bits, pre), e = row_begin(g.xadj, g.bits, pre + 1);
        for (int64_t k = b; k < e; ++k)
          if (g.adj[k] == v) { printf("[%d]\t", g.label[k]); break; }
      }
      if (j > 0) ++sampled;
      pre = v;
      printf("%d\t", v);
    }
    printf("\nTotal length=%d\n", len);
  }
  printf("Total sampled: %llu\n", sampled);
}

// src/main.cu:115-149
bool degree_bucket(int64_t n, int depth, const int32_t* result, const GraphView& g, const std::string& path) {
  std::map<int64_t, int64_t> hist;
  for (int64_t i = 0; i < n; ++i) {
    int32_t pre = -1;
    for (int j = 0; j < depth; ++j) {
      const int32_t v = result[i * depth + j];
      if (v == -1) break;
      if (pre != -1) ++hist[g.degree(pre)];
      pre = v;
    }
  }
  FILE* f = fopen(path.c_str(), "w");
  if (!f) return false;
  for (const auto& kv : hist) fprintf(f, "%lld,%lld\n", (long long)kv.first, (long long)kv.second);
  fclose(f);
  return true;
}

int fail(const char* what) {
  fprintf(stderr, "flowwalker: %s: %s\n", what, fw_last_error());
  return 1;
}

}  // namespace

int main(int argc, char** argv) {
  fwflags::Parser fl;
  define_flags(fl);
  std::string err;
  if (!fl.parse(argc, argv, &err)) { fprintf(stderr, "flowwalker: %s\n", err.c_str()); return 2; }
  if (fl.help_requested()) { fl.print_help(argv[0]); return 0; }

  const bool metapath = fl.b("metapath");
  const int apps = (int)fl.b("deepwalk") + (int)fl.b("ppr") + (int)fl.b("node2vec") + (int)metapath;
  if (apps != 1 && fl.s("save_csr").empty()) { printf("Please choose a walk mode\n"); return 0; }  // src/walk.cu:563-566
  const int app = fl.b("deepwalk") ? FW_APP_DEEPWALK : fl.b("ppr") ? FW_APP_PPR
                : fl.b("node2vec") ? FW_APP_NODE2VEC : FW_APP_METAPATH;

  // graph: weights xor labels, as include/graph.cuh:145-185
  fw_graph* g = nullptr;
  if (!fl.s("edgelist").empty()) {  // the job of data/EdgeListToCSR.cpp
    if (fw_graph_from_edgelist(fl.s("edgelist").c_str(), 5, 1.0f, 5.0f, 1, &g) != FW_OK) return fail("edge list");
  } else if (fw_graph_load(fl.s("input").c_str(), !metapath && !fl.b("lognorm"), metapath, &g) != FW_OK) {
    return fail("load");
  }
  if (!fl.s("save_csr").empty()) {
    if (fw_graph_save(g, fl.s("save_csr").c_str()) != FW_OK) return fail("save");
    printf("wrote %s_{xadj,edge,weight,label}.bin\n", fl.s("save_csr").c_str());
    fw_graph_destroy(g);
    return 0;
  }
  GraphView gv;
  fw_graph_info(g, &gv.V, &gv.E, &gv.bits, nullptr, nullptr);
  fw_graph_arrays(g, &gv.xadj, &gv.adj, &gv.weight, &gv.label);
  printf("Read Graph!\n");
  int64_t maxv = 0, maxd = 0;
  fw_graph_max_degree(g, &maxv, &maxd);
  printf("Vertex count:%lld Expected edge count: %lld\nMax degree: %lld, idx: %lld\n", (long long)gv.V,
         (long long)gv.E, (long long)maxd, (long long)maxv);
  if (fl.b("lognorm") && !metapath) {  // include/graph.cuh:79-91 (seed 1234, mean 0, sigma 3)
    std::vector<float> w((size_t)gv.E);
    if (fw_lognormal_weights(gv.E, 0.0, 3.0, 1234, w.data()) != FW_OK) return fail("lognorm");
    fw_graph* g2 = nullptr;
    if (fw_graph_from_arrays(gv.V, gv.E, gv.xadj, gv.bits, gv.adj, w.data(), nullptr, &g2) != FW_OK) return fail("lognorm");
    fw_graph_destroy(g);
    g = g2;
    fw_graph_arrays(g, &gv.xadj, &gv.adj, &gv.weight, &gv.label);
  }

  std::vector<int32_t> schema;
  if (metapath) {
    if (!parse_schema(fl.s("schema"), &schema)) { fprintf(stderr, "flowwalker: bad --schema\n"); return 2; }
    printf("schema len=%d\n", (int)schema.size());
    for (int32_t x : schema) printf("%d ", x);
    printf("\n");
  }

  // flag rewriting, src/main.cu:244-272
  int64_t n = fl.i("n");
  int d = (int)fl.i("d");
  bool seq = fl.b("seq"), batch = fl.b("batch"), autobatch = fl.b("autobatch");
  if (metapath) d = (int)schema.size();
  if (fl.b("all")) { n = gv.V; seq = true; batch = true; autobatch = true; }
  else if (fl.i("walkmode") >= 0) batch = false;
  if (autobatch) batch = true;
  if (n < 0 || d < 0) { fprintf(stderr, "flowwalker: --n and --d must be >= 0\n"); return 2; }
  const int depth = d + 1;

  // start points, src/main.cu:273-296 (seeded here)
  std::vector<int32_t> starts((size_t)n);
  if (app == FW_APP_PPR && !fl.b("uniformstarts")) {
    for (auto& s : starts) s = (int32_t)maxv;
  } else if (seq) {
    for (int64_t i = 0; i < n; ++i) starts[(size_t)i] = (int32_t)(gv.V ? i % gv.V : 0);
  } else {
    std::mt19937_64 rng((uint64_t)fl.i("startseed"));
    for (auto& s : starts) s = (int32_t)(gv.V ? rng() % (uint64_t)gv.V : 0);
  }

  fw_walk_params prm;
  memset(&prm, 0, sizeof(prm));
  prm.app = app; prm.d = d; prm.tp = fl.d("tp"); prm.p = fl.d("p"); prm.q = fl.d("q");
  prm.schema = schema.empty() ? nullptr : schema.data();
  prm.schema_len = (int32_t)schema.size();
  prm.group_mode = (int32_t)fl.i("group");
  prm.seed = (uint64_t)fl.i("seed");

  int gpus = (int)fl.i("gpus"), visible = 0;
  if (fw_device_count(&visible) != FW_OK) return fail("device count");
  if (gpus < 1 || gpus > visible) { fprintf(stderr, "flowwalker: --gpus %d but %d device(s) visible\n", gpus, visible); return 2; }

  // one engine per shard (by default one shard per GPU), queries sharded by contiguous id
  // range, graph replicated; the walks are keyed by query id, so any sharding gives the same table
  const int shards = fl.i("shards") > 0 ? (int)fl.i("shards") : gpus;
  if (shards > 64) { fprintf(stderr, "flowwalker: --shards %d is beyond 64\n", shards); return 2; }
  std::vector<int32_t> result((size_t)n * depth);
  std::vector<fw_walk_stats> stats((size_t)shards);
  std::vector<int> rcs((size_t)shards, FW_OK);
  std::vector<std::string> errs((size_t)shards);
  std::vector<fw_engine*> engines((size_t)shards, nullptr);
  for (int r = 0; r < shards; ++r)
    if (fw_engine_create(g, r % gpus, fl.b("umgraph") ? FW_ENGINE_MANAGED : 0, &engines[(size_t)r]) != FW_OK) return fail("engine");
  const auto t0 = std::chrono::steady_clock::now();
  std::vector<std::thread> threads;
  for (int r = 0; r < shards; ++r) {
    threads.emplace_back([&, r]() {
      if (fl.b("interleave") && shards > 1) {
        // ids r, r + S, ...: gather the shard's start points, walk, scatter its rows back
        const int64_t m = n > r ? (n - r + shards - 1) / shards : 0;
        std::vector<int32_t> st((size_t)m), res((size_t)m * depth);
        for (int64_t i = 0; i < m; ++i) st[(size_t)i] = starts[(size_t)(r + i * shards)];
        fw_walk_params p = prm;
        p.query_id_base = (uint64_t)r;
        p.query_id_stride = (uint64_t)shards;
        const int rc = fw_walk(engines[(size_t)r], &p, st.data(), m, res.data(), &stats[(size_t)r], nullptr);
        if (rc == FW_OK)
          for (int64_t i = 0; i < m; ++i)
            memcpy(result.data() + (size_t)(r + i * shards) * depth, res.data() + (size_t)i * depth, (size_t)depth * 4);
        rcs[(size_t)r] = rc;
        if (rc != FW_OK) errs[(size_t)r] = fw_last_error();
        return;
      }
      const int64_t lo = r * n / shards, hi = (r + 1) * n / shards;
      fw_walk_params p = prm;
      p.query_id_base = (uint64_t)lo;
      int rc;
      if (batch) {
        int32_t* pinned = nullptr;
        rc = fw_walk_batch(engines[(size_t)r], &p, starts.data() + lo, hi - lo, autobatch ? 0 : fl.i("batchsize"),
                           (int32_t)fl.i("headroom"), &pinned, &stats[(size_t)r], nullptr);
        if (rc == FW_OK && hi > lo) memcpy(result.data() + (size_t)lo * depth, pinned, (size_t)(hi - lo) * depth * 4);
        fw_free_pinned(pinned);
      } else {
        rc = fw_walk(engines[(size_t)r], &p, starts.data() + lo, hi - lo, result.data() + (size_t)lo * depth,
                     &stats[(size_t)r], nullptr);
      }
      rcs[(size_t)r] = rc;
      if (rc != FW_OK) errs[(size_t)r] = fw_last_error();
    });
  }
  for (auto& t : threads) t.join();
  const double wall_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  for (int r = 0; r < shards; ++r) {
    if (rcs[(size_t)r] != FW_OK) { fprintf(stderr, "flowwalker: walk of shard %d on GPU %d: %s\n", r, r % gpus, errs[(size_t)r].c_str()); return 1; }
  }
  uint64_t steps = 0, scanned = 0;
  double dev_ms = 0;
  uint32_t status = 0;
  for (const auto& s : stats) {
    steps += s.steps; scanned += s.scanned; status |= s.device_status;
    if (s.device_ms > dev_ms) dev_ms = s.device_ms;
  }
  printf("sampling time:%.6f ms (device, max over %d GPU%s); end to end %.6f ms\n", dev_ms, gpus, gpus > 1 ? "s" : "", wall_ms);
  printf("{\"app\": %d, \"n\": %lld, \"d\": %d, \"gpus\": %d, \"steps\": %llu, \"scanned\": %llu, \"device_ms\": %.6f, "
         "\"steps_per_s\": %.6g, \"device_status\": %u}\n",
         app, (long long)n, d, gpus, (unsigned long long)steps, (unsigned long long)scanned, dev_ms,
         dev_ms > 0 ? steps / (dev_ms * 1e-3) : 0.0, status);

  if (fl.b("printresult")) {
    if (metapath) print_res_metapath(n, depth, result.data(), gv); else print_res(n, depth, result.data());
  }
  if (fl.b("printworkload")) {  // src/main.cu:82-113
    printf("Total sampled vertex: %llu\n", (unsigned long long)steps);
    printf("Total sampled edge: %llu,throughput: %f edges per s\n", (unsigned long long)scanned,
           dev_ms > 0 ? scanned / (dev_ms * 1e-3) : 0.0);
  }
  if (fl.b("save_degree") && !degree_bucket(n, depth, result.data(), gv, fl.s("b_file")))
    fprintf(stderr, "flowwalker: cannot write %s\n", fl.s("b_file").c_str());
  if (!fl.s("save_result").empty()) {
    FILE* f = fopen(fl.s("save_result").c_str(), "wb");
    if (!f || fwrite(result.data(), 4, result.size(), f) != result.size()) { fprintf(stderr, "flowwalker: cannot write %s\n", fl.s("save_result").c_str()); return 1; }
    fclose(f);
  }
  for (fw_engine* e : engines) fw_engine_destroy(e);
  fw_graph_destroy(g);
  return status ? 3 : 0;
}
