// Harness around the UNMODIFIED reference walker (its src/walk.cu, src/util.cu and include/
// headers are compiled where they lie; nothing of them is copied here).  It feeds the
// reference's own loader (include/graph.cuh:93-190) a CSR written by this repo's generator,
// calls the reference's walk_test (src/walk.cu:527-574) exactly as its main does
// (src/main.cu:348-358), reports the time the reference itself measures and dumps the whole
// result pool, which the stock CLI cannot do (it prints 100 walks, src/main.cu:165).
// Test and baseline infrastructure only: the product never links this.
//
//   ref_walk <prefix> <deepwalk|ppr|node2vec|metapath> <d> <starts.bin> <n> <out.bin|-> [tp p q] [schema csv]
// Environment: FW_REF_REPEAT=k repeats the walk k times (one REFJSON line each, the last
// result is the one dumped); FW_REF_BATCH=1 calls walk_batch (src/walk.cu:576-649: pinned
// host result, copies inside its timed region) instead of walk_test.
#include <cuda_runtime.h>
#include <gflags/gflags.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "walker.cuh"

// the flags the reference's translation units declare
// (src/walk.cu:36-44, include/gpu_graph.cuh:25-26, include/graph.cuh:35-36)
DEFINE_double(tp, 0.2, "");
DEFINE_double(p, 2.0, "");
DEFINE_double(q, 0.5, "");
DEFINE_bool(deepwalk, false, "");
DEFINE_bool(ppr, false, "");
DEFINE_bool(node2vec, false, "");
DEFINE_bool(metapath, false, "");
DEFINE_bool(syn, false, "");
DEFINE_bool(dprs, false, "");
DEFINE_bool(umgraph, false, "");
DEFINE_bool(lognorm, false, "");

int main(int argc, char** argv) {
  if (argc < 7) {
    fprintf(stderr, "usage: %s prefix app d starts.bin n out.bin|- [tp p q] [schema]\n", argv[0]);
    return 2;
  }
  const std::string prefix = argv[1], app = argv[2];
  const int d = atoi(argv[3]);
  const char* starts_path = argv[4];
  const int n = atoi(argv[5]);
  const char* out_path = argv[6];
  if (argc > 9) { FLAGS_tp = atof(argv[7]); FLAGS_p = atof(argv[8]); FLAGS_q = atof(argv[9]); }
  std::vector<int> schema;
  if (argc > 10) {
    char* tok = strtok(argv[10], ",");
    while (tok) { schema.push_back(atoi(tok)); tok = strtok(nullptr, ","); }
  }
  FLAGS_deepwalk = app == "deepwalk";
  FLAGS_ppr = app == "ppr";
  FLAGS_node2vec = app == "node2vec";
  FLAGS_metapath = app == "metapath";
  FLAGS_dprs = FLAGS_node2vec;  // the production (batch) path picks the one-loop sampler for node2vec: src/walk.cu:403-406
  if (!(FLAGS_deepwalk || FLAGS_ppr || FLAGS_node2vec || FLAGS_metapath)) { fprintf(stderr, "unknown app\n"); return 2; }

  graph* ginst = new graph((prefix + "_xadj.bin").c_str(), (prefix + "_edge.bin").c_str(),
                           (prefix + "_weight.bin").c_str(), (prefix + "_label.bin").c_str());
  gpu_graph* ggraph = new gpu_graph(ginst);

  vtx_t* starts = nullptr;
  if (cudaMallocHost(&starts, sizeof(vtx_t) * (size_t)n) != cudaSuccess) { fprintf(stderr, "cudaMallocHost failed\n"); return 1; }
  FILE* f = fopen(starts_path, "rb");
  if (!f || fread(starts, sizeof(vtx_t), (size_t)n, f) != (size_t)n) { fprintf(stderr, "cannot read %s\n", starts_path); return 1; }
  fclose(f);

  const int depth = d + 1;  // src/main.cu:339
  const int repeat = getenv("FW_REF_REPEAT") ? atoi(getenv("FW_REF_REPEAT")) : 1;
  const bool batch = getenv("FW_REF_BATCH") && atoi(getenv("FW_REF_BATCH")) != 0;
  const size_t cells = (size_t)n * depth;
  std::vector<vtx_t> host;
  const vtx_t* walks = nullptr;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  for (int rep = 0; rep < repeat; ++rep) {
    vtx_t* result = nullptr;
    cudaEventRecord(e0);
    const double ref_ms =
        batch ? walk_batch(result, ggraph, starts, depth, n, n, schema.empty() ? nullptr : schema.data(), (int)schema.size())
              : walk_test(result, ggraph, starts, depth, n, wb_dynamic, schema.empty() ? nullptr : schema.data(),
                          (int)schema.size());
    cudaEventRecord(e1);
    cudaEventSynchronize(e1);
    float ev_ms = 0.f;
    cudaEventElapsedTime(&ev_ms, e0, e1);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) { fprintf(stderr, "CUDA error after the walk: %s\n", cudaGetErrorString(err)); return 1; }
    if (batch) {
      walks = result;  // pinned host memory (src/walk.cu:586)
    } else {
      host.resize(cells);
      cudaMemcpy(host.data(), result, cells * sizeof(vtx_t), cudaMemcpyDeviceToHost);
      cudaFree(result);
      walks = host.data();
    }
    unsigned long long steps = 0, scanned = 0;  // as calculate_workload, src/main.cu:93-109
    for (int i = 0; i < n; ++i) {
      vtx_t pre = -1;
      for (int j = 0; j < depth; ++j) {
        const vtx_t v = walks[(size_t)i * depth + j];
        if (v == -1) break;
        if (j > 0) ++steps;
        if (pre != -1) scanned += ginst->xadj[pre + 1] - ginst->xadj[pre];
        pre = v;
      }
    }
    printf("REFJSON {\"app\": \"%s\", \"n\": %d, \"d\": %d, \"batch\": %d, \"ref_ms\": %.6f, \"event_ms\": %.6f, \"steps\": %llu, \"scanned\": %llu}\n",
           app.c_str(), n, d, batch ? 1 : 0, ref_ms, ev_ms, steps, scanned);
    fflush(stdout);
    if (batch && rep + 1 < repeat) cudaFreeHost(result);
  }
  if (strcmp(out_path, "-") != 0) {
    FILE* o = fopen(out_path, "wb");
    if (!o || fwrite(walks, sizeof(vtx_t), cells, o) != cells) { fprintf(stderr, "cannot write %s\n", out_path); return 1; }
    fclose(o);
  }
  return 0;
}
