/*
 * flowwalker.h -- C ABI of the B200 random-walk engine.
 *
 * Plain C types only: pointers, sizes and PODs.  Every function returns an
 * int status (FW_OK = 0, negative = error; the message is available from
 * fw_last_error() on the calling thread) and never calls exit().  Calls on one engine from
 * several threads are serialised inside the library; different engines run concurrently.  Objects
 * created by a *_create / *_load / *_generate call are released by the matching
 * *_destroy.  Buffers passed in stay owned by the caller.
 *
 * The reference program has no FFI of its own; its operator surface for the
 * walk path is (a) the on-disk CSR format, (b) the two host entry points
 * walk_test / walk_batch, (c) the four device-side "walker" classes and (d)
 * the command-line flags.  Each declaration below names the part of the
 * reference it stands in for (path:line inside the reference project).
 */
#ifndef FLOWWALKER_H_
#define FLOWWALKER_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FW_OK 0
#define FW_ERR_ARG (-1)     /* bad argument */
#define FW_ERR_IO (-2)      /* missing / truncated / inconsistent file */
#define FW_ERR_CUDA (-3)    /* a CUDA runtime call failed */
#define FW_ERR_NOMEM (-4)   /* host or device allocation failed */
#define FW_ERR_DEVICE (-5)  /* the kernel gave up on a bounded wait (FW_STATUS_WAIT_TIMEOUT): result incomplete */

/* Applications: include/app.cuh:58-152 (Deepwalk, PPR, Node2vec, Metapath). */
#define FW_APP_DEEPWALK 0
#define FW_APP_PPR 1
#define FW_APP_NODE2VEC 2
#define FW_APP_METAPATH 3

/* Sampler granularity: how many neighbours share one exponential key. */
#define FW_GROUP_EDGE 1    /* one key per neighbour */
#define FW_GROUP_STRIP 64  /* one key per strip of up to 64 neighbours (default) */

/* Bits of fw_walk_stats.device_status (0 = clean run). */
#define FW_STATUS_BAD_START 1u     /* a start vertex outside [0,V) (walk has 0 steps) */
#define FW_STATUS_BAD_NEIGHBOR 2u  /* a neighbour id outside [0,V) (walk ended there) */
#define FW_STATUS_WAIT_TIMEOUT 4u  /* a bounded wait on a staged copy ran out */

typedef struct fw_graph fw_graph;   /* host CSR: include/graph.cuh:44-51 */
typedef struct fw_engine fw_engine; /* device CSR replica on one GPU: include/gpu_graph.cuh:28-78 */

/*
 * Walk parameters.  Stands in for the constructor arguments of the walker
 * classes (include/app.cuh:47-50, 78-82, 102-107, 135-140) and the flags that
 * feed them (src/main.cu:43, 54-58).  `d` is the number of steps (--d); the
 * result has d+1 columns, which is what the reference calls max_depth.
 */
typedef struct fw_walk_params {
  int32_t app;            /* FW_APP_* */
  int32_t d;              /* steps per walk; MetaPath callers pass the schema length */
  double tp;              /* PPR: stop probability after every step (--tp) */
  double p;               /* node2vec return parameter (--p) */
  double q;               /* node2vec in-out parameter (--q) */
  const int32_t* schema;  /* MetaPath: edge label wanted at step k is schema[k % schema_len] */
  int32_t schema_len;
  int32_t group_mode;     /* FW_GROUP_*; 0 selects the default */
  uint64_t seed;          /* Philox key; the reference hard-codes 1337 (include/walker.cuh:1324) */
  uint64_t query_id_base; /* global id of starts[0]; walk i is keyed by query_id_base + i * stride */
  uint64_t query_id_stride; /* distance between the global ids of consecutive queries; 0 means 1.
                             * Rank r of R walking the ids r, r+R, r+2R, ... of one job (an
                             * interleaved shard) passes base = r, stride = R. */
} fw_walk_params;

typedef struct fw_walk_stats {
  uint64_t steps;         /* result cells != -1 beyond column 0 (src/main.cu:103) */
  uint64_t scanned;       /* sum of out-degrees stepped from (src/main.cu:104-105) */
  double device_ms;       /* CUDA-event time of the walk kernel(s) only */
  double total_ms;        /* fw_walk only: copies + kernel, event-timed on the engine's stream */
  uint32_t device_status; /* FW_STATUS_* bits */
  uint32_t launches;      /* kernel launches issued by this call */
} fw_walk_stats;

/* R-MAT generator parameters (stand-in for the datasets of data/get_dataset.sh). */
typedef struct fw_rmat_params {
  int32_t scale;          /* ids have `scale` bits */
  int32_t xadj_bits;      /* 32 or 64 */
  int64_t draws;          /* candidate edges drawn (scale-22 edge factor 16: 16 << 22) */
  double a, b, c;         /* quadrant probabilities (d = 1-a-b-c) */
  uint64_t seed;          /* graph seed */
  int64_t v_limit;        /* > 0: vertex count; candidates touching ids >= v_limit are dropped */
  int64_t e_target;       /* > 0: keep drawing (beyond `draws`) until exactly this many distinct edges */
  float weight_lo, weight_hi; /* weights uniform in [lo, hi); lo == hi == 0 -> no weights */
  uint64_t weight_seed;
  int32_t n_labels;       /* labels uniform in {0..n_labels-1}; 0 -> no labels */
  uint64_t label_seed;
  int32_t device;         /* >= 0: generate on that GPU; -1: on the host */
} fw_rmat_params;

const char* fw_last_error(void);
/* Revision tag of the walk kernels (changes whenever their code does): profile-derived figures
 * quoted beside a measurement name the revision they were captured on. */
const char* fw_kernel_revision(void);
/* Number of CUDA devices visible to the process. */
int fw_device_count(int* count);

/* ---- graph: on-disk format of include/graph.cuh:93-190, writer data/EdgeListToCSR.cpp:217-251 ---- */

/* Reads <prefix>_xadj.bin, _edge.bin and, as asked, _weight.bin / _label.bin.
 * The reference reads weights xor labels depending on --metapath
 * (include/graph.cuh:145-185).  A 64-bit offset file (8-byte header followed
 * by int64 offsets) is recognised by its size. */
int fw_graph_load(const char* prefix, int need_weight, int need_label, fw_graph** out);
int fw_graph_save(const fw_graph* g, const char* prefix);
/* Copies the arrays.  xadj_bits: 32 (uint32) or 64 (int64). weight / label may be NULL. */
int fw_graph_from_arrays(int64_t V, int64_t E, const void* xadj, int xadj_bits,
                         const int32_t* adj, const float* weight,
                         const int32_t* label, fw_graph** out);
int fw_rmat_generate(const fw_rmat_params* params, fw_graph** out);
/* Text edge list ("u v" per line, '#' or '%' comments) -> undirected, deduplicated CSR with vertices
 * renumbered by first appearance and one label / weight per undirected edge, as the reference's
 * converter does (data/EdgeListToCSR.cpp:132-268); rows sorted, self-loops dropped, attributes seeded. */
int fw_graph_from_edgelist(const char* path, int32_t n_labels, float weight_lo, float weight_hi,
                           uint64_t seed, fw_graph** out);
/* Seeded log-normal edge weights, the job of --lognorm (include/graph.cuh:79-91: mean 0, sigma 3,
 * seed 1234 there, drawn with cuRAND).  out[i] = exp(mean + sigma * z_i), z_i a standard normal
 * formed by the Box-Muller transform from Philox4x32-10 block i / 2 keyed by `seed`; computed in
 * double precision and rounded to float, so the values depend on the seed only. */
int fw_lognormal_weights(int64_t n, double mean, double sigma, uint64_t seed, float* out);
int fw_graph_info(const fw_graph* g, int64_t* V, int64_t* E, int32_t* xadj_bits,
                  int32_t* has_weight, int32_t* has_label);
/* Borrowed pointers into the graph (valid until fw_graph_destroy). */
int fw_graph_arrays(const fw_graph* g, const void** xadj, const int32_t** adj,
                    const float** weight, const int32_t** label);
/* Index of the vertex of largest out-degree (include/graph.cuh get_maxdegree_offset,
 * used for the PPR start points in src/main.cu:277-281). */
int fw_graph_max_degree(const fw_graph* g, int64_t* vertex, int64_t* degree);
void fw_graph_destroy(fw_graph* g);

/* ---- engine: gpu_graph construction (include/gpu_graph.cuh:39-78) ---- */

/* Uploads (replicates) the graph to `device`.  which: bit 0 = weights, bit 1 = labels; neither
 * bit uploads whatever the graph has.  FW_ENGINE_MANAGED (bit 2) puts the edge arrays in unified
 * memory (the role of --umgraph, include/gpu_graph.cuh:46-54): they may then exceed the device's
 * memory, live on the device as far as they fit and migrate on demand. */
#define FW_ENGINE_MANAGED 4
int fw_engine_create(const fw_graph* g, int device, int which, fw_engine** out);
void fw_engine_destroy(fw_engine* e);
int fw_engine_device(const fw_engine* e, int* device, int* sm_count);
/* Block-granularity sampling of very long rows (the role of sampler_block, include/sampler.cuh:87-127):
 * warps that ran out of queries help the warps of their CTA that sit on rows of 32,768+ edges.
 * mode -1 (default): on for DeepWalk, PPR and MetaPath on graphs whose largest out-degree is
 * >= 262,144; 0: off; 1: on for every app.
 * Results do not depend on it. */
int fw_engine_set_sharing(fw_engine* e, int mode);
/* Hub batching (the other half of the role of sampler_block, include/sampler.cuh:87-127, and of
 * the degree-binned dispatch of include/walker.cuh:1357-1419): walkers that arrive at a vertex of
 * about a thousand neighbours or more (1,016; 504 in calls with many queries per such vertex)
 * wait there, and one sweep of the hub's row serves up to 32 of them.
 * All four applications with the strip sampler (MetaPath: walkers that want the same label share;
 * node2vec: the sweep of plain weights is shared, every walker's bias test is its own); a walk
 * call then is a series of kernel launches.
 * mode -1 (default): on when the graph has such vertices and the call brings enough queries per
 * hub of 1,016 neighbours or more to earn back the fixed cost of the series (64 or more); 0: off;
 * 1: on whenever the graph has hubs; 2: as 1, and batching down to the last walker (by default
 * the last parked walkers of a call are walked to the end by one launch without batching).
 * Results do not depend on it. */
int fw_engine_set_hub_batching(fw_engine* e, int mode);
/* Early delivery of the walk table (the role of the reference's overlap of walking and copying in
 * walk_batch, src/walk.cu:373-466, inside one call): when the result buffer of fw_walk,
 * fw_walk_batch or fw_walk_batch_into is page-locked host memory the device can address
 * (cudaHostAlloc, cudaMallocHost, cudaHostRegister; fw_walk_batch's own buffer always is), the
 * call is hub-batched and a result row has at least 32 cells, the rows of walks that have ended
 * are written to it by a small kernel on a stream of its own while the remaining walkers walk on,
 * instead of one copy of the whole table after the last launch.
 * mode -1 (default): delivery begins once the call has run for a quarter of the time its table
 * needs on the host link, so a call whose walk is short beside its copy never delivers, and a call
 * that ends with less than a quarter of its rows delivered stops delivering and copies the table
 * in one piece; 0: never (one copy at the end); 1: from the first launch on, to the last row;
 * 2: from the first launch on, then always the fallback copy (1 and 2 exist for tests).
 * The environment variable FLOWWALKER_EARLY_DELIVERY=0 has the effect of mode 0.
 * Results do not depend on it. */
int fw_engine_set_early_delivery(fw_engine* e, int mode);
/* Number of hub vertices of the engine's graph and the row length from which a vertex is one,
 * for the two limits a call chooses from (which = 0: 1,016 neighbours, 1: 504; the lower one
 * serves calls that bring at least a hundred queries per hub). */
int fw_engine_hubs(const fw_engine* e, int which, int32_t* n_hubs, uint32_t* min_degree);

/*
 * walk_test (include/walker.cuh:49-52, src/walk.cu:527-574): start points on
 * the host, result left on the device.  Here the caller owns both device
 * buffers: starts_dev int32[n], result_dev int32[n*(d+1)] (fully written,
 * -1 padded; no memset needed).  `stream` is a cudaStream_t (NULL = the
 * engine's own stream).  Returns after the kernel has finished.  len_hist
 * (optional, host) receives d+1 walk-length counts.
 */
int fw_walk_device(fw_engine* e, const fw_walk_params* params,
                   const int32_t* starts_dev, int64_t n, int32_t* result_dev,
                   void* stream, fw_walk_stats* stats, uint64_t* len_hist);

/*
 * Host-buffer form of the same call: copies starts_host to the device, walks,
 * copies the result back into result_host (int32[n*(d+1)]).  total_ms covers
 * both copies and the kernel.
 */
int fw_walk(fw_engine* e, const fw_walk_params* params, const int32_t* starts_host,
            int64_t n, int32_t* result_host, fw_walk_stats* stats, uint64_t* len_hist);

/*
 * walk_batch (include/walker.cuh:54-57, src/walk.cu:373-466, 576-649): walks
 * n queries in batches of batch_size on two streams, double-buffered, each
 * batch's result copied to pinned host memory while the next one runs.
 * *result_pinned is allocated by the callee with cudaMallocHost as in the
 * reference (src/walk.cu:586); release it with fw_free_pinned.  batch_size <= 0
 * picks a size from free device memory minus headroom_mb, as --autobatch does
 * (src/main.cu:259-271).
 */
int fw_walk_batch(fw_engine* e, const fw_walk_params* params, const int32_t* starts_host,
                  int64_t n, int64_t batch_size, int32_t headroom_mb,
                  int32_t** result_pinned, fw_walk_stats* stats, uint64_t* len_hist);
void fw_free_pinned(void* p);
/* The same double-buffered pipeline into a host buffer the caller owns (int32[n*(d+1)]; page-locked
 * memory lets the device-to-host copy of one batch overlap the walk of the next).  Stands in for
 * timing_batch_async (src/walk.cu:373-466) without its allocation. */
int fw_walk_batch_into(fw_engine* e, const fw_walk_params* params, const int32_t* starts_host,
                       int64_t n, int64_t batch_size, int32_t headroom_mb,
                       int32_t* result_host, fw_walk_stats* stats, uint64_t* len_hist);

/*
 * Failure-detection self-test, no counterpart in the reference (whose device waits are
 * unbounded and whose host code exits on any CUDA error, include/util.cuh:56-68).  One warp
 * waits on a barrier that nothing completes, with the same bounded polling loop the staging
 * ring uses and `polls` as the limit; *status receives FW_STATUS_WAIT_TIMEOUT and the context
 * stays usable.
 */
int fw_selftest_wait_timeout(int device, uint32_t polls, uint32_t* status);

/*
 * Allocation-free walk.  No counterpart in the reference (its host code
 * allocates at every call, src/walk.cu:98-138, 586).
 *
 * For callers that cannot allocate device memory when they call: a plugin
 * living inside another framework's memory pool that already owns the GPU, a
 * serving loop that must not hit the device-wide synchronisation of
 * cudaMalloc/cudaFree, a process whose allocator is frozen after start-up.
 * The caller passes the CSR, the start points and the result as device
 * pointers on `device`; the walk's scratch (query counter, counters,
 * walk-length histogram) is a fixed 32 KB array inside the loaded module, so
 * this call performs no cudaMalloc, cudaFree or other allocating call.
 *
 * Limits and rules:
 *  - d <= 4095 (larger values are rejected with FW_ERR_ARG: use fw_walk_device);
 *    device ordinal < 64 and visible, compute capability >= 10; schema_len <= 64.
 *  - xadj_dev holds V + 1 row offsets (32- or 64-bit as xadj_bits says).
 *    adj_dev / weight_dev / label_dev must be 16-byte aligned and readable up
 *    to the next multiple of 4 elements past E (the kernel reads whole
 *    16-byte quads); weight_dev may be NULL for MetaPath, label_dev otherwise.
 *    node2vec needs every row of adj_dev sorted ascending (its membership test
 *    is a binary search, as include/gpu_graph.cuh:97-118).
 *  - `stream` is a cudaStream_t; NULL here is the legacy default stream (not an
 *    engine's own stream as in fw_walk_device: there is no engine).
 *  - The first call on each device is a set-up call: it looks up the scratch
 *    address (cudaGetSymbolAddress) and, with lazy module loading, may make
 *    the driver load the kernel (which allocates inside the driver).  Make
 *    that first call at start-up, outside any stream capture.  The promise
 *    "no allocating call" holds for every call after it.
 *  - All calls on one device share the scratch array, which keeps the last
 *    call's contents; each call clears what it uses, so calls must not overlap
 *    on the GPU (two streams, or two host threads on the same device, race).
 *  - The call synchronises `stream` and returns after the kernel has finished
 *    (counters travel back by plain copies); stats->device_ms / total_ms are
 *    not measured (0) since events would have to be created.  stats and
 *    len_hist (host, d+1 words) may be NULL.
 */
int fw_walk_csr_noalloc(int device, int64_t V, int64_t E, const void* xadj_dev, int xadj_bits,
                        const int32_t* adj_dev, const float* weight_dev, const int32_t* label_dev,
                        const fw_walk_params* params, const int32_t* starts_dev, int64_t n,
                        int32_t* result_dev, void* stream, fw_walk_stats* stats, uint64_t* len_hist);

#ifdef __cplusplus
}
#endif
#endif /* FLOWWALKER_H_ */
