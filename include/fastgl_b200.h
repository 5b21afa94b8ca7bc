/*
 * fastgl_b200 -- C ABI of the B200 (sm_100a) implementation of FastGL's per-mini-batch hot path:
 * CSR neighbour sampling, the Fused-Map id mapping, block-CSR helpers and sum / mean / sym-norm
 * aggregation (forward and backward).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (a cudaStream_t passed as
 * void*; NULL = the legacy default stream) and returns an int status (FGL_OK = 0).  Nothing here
 * includes or names a PyTorch type.  All index arrays are int32 unless stated; feature matrices are
 * fp32, row-major, with an explicit leading dimension in elements.  Unless a function says otherwise
 * it only enqueues work on the stream and returns without synchronising.
 *
 * Each declaration cites the interface of the reference (cuda_operators/..., file:line) that it
 * replaces.  The dense weight products that the reference performs inside its ops (torch::mm) are
 * not part of this library; the host language keeps them (cuBLAS through PyTorch).
 */
#ifndef FASTGL_B200_H_
#define FASTGL_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FGL_ABI_VERSION 3

/* status codes */
#define FGL_OK 0
#define FGL_ERR_INVALID 1  /* bad argument (null pointer, negative size, unsupported fanout ...) */
#define FGL_ERR_CUDA 2     /* a CUDA runtime call failed; see fgl_last_error() */
#define FGL_ERR_NOMEM 3    /* workspace allocation failed */
#define FGL_ERR_CAPACITY 4 /* an output buffer or the hashtable is too small for the result */
#define FGL_ERR_PROBE 5    /* hashtable probe limit reached (table full or corrupted) */
#define FGL_ERR_BOUNDS 6   /* a node id outside [0, n_nodes) was met on the device */
#define FGL_ERR_TIMEOUT 7  /* a bounded device-side wait gave up */

/* flags of fgl_sample / fgl_sample_map_fused */
#define FGL_SAMPLE_REPLACE 1   /* hubs (deg > fanout): independent picks, duplicates possible (reference) */
/* flags of fgl_map / fgl_sample_map_fused */
#define FGL_MAP_ARRIVAL_ORDER 2 /* new ids in atomic arrival order (reference) instead of first occurrence */
/* flags of fgl_agg_fwd */
#define FGL_AGG_ZERO_DEG_PASSTHROUGH 1 /* a row without in-edges copies its own input row (reference) */

/* aggregation modes */
#define FGL_AGG_SUM 0     /* out[d] = sum_s x[s]                                  (GIN,  K10/K11) */
#define FGL_AGG_MEAN 1    /* out[d] = sum_s x[s] / deg_in(d)                      (GraphSAGE-mean) */
#define FGL_AGG_SYMNORM 2 /* out[d] = sum_s x[s] * rsqrt(dst_deg[d]) * rsqrt(src_deg[s]) (GCN, K8/K9) */
#define FGL_AGG_EDGE 3    /* out[d, h] = sum_e w[e, h] * x[src[e], h]: per-edge, per-head weights (GAT, K12);
                             only through fgl_agg_edge_fwd / fgl_agg_edge_bwd */

/* flags of fgl_bias_relu_dropout / fgl_relu_dropout_bwd */
#define FGL_EW_RELU 1     /* apply ReLU (forward) / the ReLU-and-dropout mask (backward) */

#define FGL_MAX_HOPS 7
#define FGL_COUNTS_STRIDE 16 /* per mini-batch: [0..7] node counts n_0..n_L, [8..15] edge counts per hop */
#define FGL_MAX_FANOUT 512

typedef struct fgl_ws fgl_ws; /* per-device workspace: hashtable, scan scratch, status words */

int fgl_abi_version(void);
int fgl_sizeof_fused_args(void); /* sizeof(struct fgl_fused_args), for bindings to check their layout */
const char* fgl_status_str(int status);

/* Workspace.  Replaces the per-call cudaMalloc / cudaFree of scratch in the reference
 * (sample.cu:118,151,157,161-162,197; id_map.cu:45-58; utilis.cu:33,38).  Buffers grow on demand
 * (never inside a stream capture: size the workspace with fgl_ws_reserve first) and are freed by
 * fgl_ws_destroy.  A workspace belongs to one device and may be used from any host thread: the lock a call
 * takes only covers its enqueueing.  The kernels of one workspace share its table, scratch, barrier and
 * status words, so calls on one workspace must be stream-ordered (one stream, or streams the caller orders
 * with events); calls that may overlap on the GPU need a workspace each. */
int fgl_ws_create(int device, fgl_ws** ws);
int fgl_ws_destroy(fgl_ws* ws);
int fgl_ws_reserve(fgl_ws* ws, int64_t table_slots, int64_t scratch_bytes);
const char* fgl_last_error(fgl_ws* ws);
/* Reads back (synchronising the stream) and clears the device status word set by the kernels of this
 * workspace: FGL_OK or the first FGL_ERR_* a kernel recorded. */
int fgl_ws_check(fgl_ws* ws, void* stream);
/* Enqueues a copy of the status word to host_dst (pinned host memory, one int32) on the stream, without
 * synchronising and without clearing it: a caller that already waits for another read-back of the same stream
 * learns of device-side errors at that point for free.  After a non-zero value, fgl_ws_check clears the word. */
int fgl_ws_status_peek(fgl_ws* ws, int32_t* host_dst, void* stream);

/* Measurement aid: the next launch of fgl_sample_map_fused, fgl_map or fgl_agg_fwd_window on this workspace records
 * the two CUDA events (cudaEvent_t, created with timing enabled) on its stream directly before and after its
 * kernel launch, then forgets them.  Events recorded by the caller around the call would also cover the call's
 * host-side preparation whenever the GPU is idle at that moment.  Pass two null pointers to cancel. */
int fgl_ws_time_next_launch(fgl_ws* ws, void* start_event, void* end_event);

/* Self-test of the library's bounded device-side wait (no counterpart in the reference, whose kernels never
 * wait on one another): n_ctas (<= 64) CTAs arrive at a barrier that expects n_ctas + 1 arrivals, so every wait
 * gives up after spin_limit polls, records FGL_ERR_TIMEOUT and raises the workspace's abort flag.  Nothing
 * faults and nothing hangs; the next fgl_ws_check returns FGL_ERR_TIMEOUT and clears the flag, after which the
 * workspace works as before. */
int fgl_selftest_barrier_timeout(fgl_ws* ws, int32_t n_ctas, int64_t spin_limit, void* stream);

/* Measurement probe (no counterpart in the reference): launches a kernel that performs the sampler's memory access
 * pattern and nothing else -- per access one 4-byte read at a hashed position of array[n_words] (the cost of
 * picking a neighbour in a long adjacency list) and, if table is given (table_slots 64-bit words, a power of two,
 * zero-filled by the caller), a dependent load of a hashed slot plus a compare-and-swap when it looks empty (the
 * first probe of the id map's insert).  Every thread of 2 CTAs x 512 threads per SM keeps four chains in flight
 * for iters rounds; *n_accesses receives the number of accesses the launch performs, so that the caller, timing
 * the stream, gets accesses per second: the roofline of the fused sampler by access count rather than by bytes.
 * sink: one int32 of device memory the kernel may write. */
int fgl_probe_access_pattern(const int32_t* array, int64_t n_words, uint64_t* table, int64_t table_slots, int32_t iters,
                             int32_t* sink, int64_t* n_accesses, void* stream);

/* Neighbour sampling; replaces sample_node_cuda (sample.cu:102-203; binding aggregate_acc.cpp:491-512).
 * indptr has n_nodes + 1 entries of int32 (indptr_is_64 = 0, as the reference) or int64.  For seed i
 * the k_i = min(deg, fanout) sampled sources land at out_src[out_indptr[i] .. out_indptr[i+1]); a seed
 * with deg <= fanout gets its whole list in CSR order.  out_src needs n_seeds * fanout entries.
 * out_dst (may be NULL) receives the seed's global id per edge, out_indptr (may be NULL only if the
 * caller does not need the block CSR) the n_seeds + 1 offsets.  Random picks come from Philox4x32-10
 * with key = rng_seed and counter = (pick slot, seed position, rng_ctr): the same arguments give the
 * same edges.  If n_edges_host is not NULL the call synchronises the stream, stores the edge count
 * there and returns the device status. */
int fgl_sample(fgl_ws* ws, const void* indptr, int indptr_is_64, const int32_t* indices, int64_t n_nodes,
               const int32_t* seeds, int32_t n_seeds, int32_t fanout, int32_t flags, uint64_t rng_seed,
               uint64_t rng_ctr, int32_t* out_indptr, int32_t* out_src, int32_t* out_dst,
               int64_t* n_edges_host, void* stream);

/* Fused-Map id mapping; replaces transfer_edge_id_cuda (id_map.cu:386-493; binding
 * aggregate_acc.cpp:467-489).  src (and dst, if not NULL) hold global ids on entry and block-local ids
 * on return (in place, like the reference).  unique receives the n_seeds seeds followed by every
 * source that is not a seed, each once: in first-occurrence order of src, or with
 * FGL_MAP_ARRIVAL_ORDER in whatever order the inserting threads arrive (the reference's behaviour).
 * unique_cap is the capacity of unique in entries.  If n_unique_host is not NULL the call
 * synchronises, stores the total number of unique nodes and returns the device status. */
int fgl_map(fgl_ws* ws, int32_t* src, int32_t* dst, const int32_t* seeds, int32_t n_seeds, int64_t n_edges,
            int32_t* unique, int64_t unique_cap, int32_t flags, int64_t* n_unique_host, void* stream);

/* Multi-hop, multi-mini-batch sampling + mapping in one persistent kernel; replaces the per-hop loop
 * sample_node -> transfer_edge_id of FusedMapSampler.sample_blocks (FusedMapSampler.py:72-109) for
 * n_batches independent mini-batches at once.  All pointers are device pointers. */
typedef struct fgl_fused_args {
    const void* indptr;         /* n_nodes + 1 entries */
    const int32_t* indices;
    int64_t n_nodes;
    int32_t indptr_is_64;
    int32_t n_batches;
    int32_t n_hops;                /* 1 .. FGL_MAX_HOPS */
    int32_t fanout[FGL_MAX_HOPS];  /* in sampling order: fanout[0] is applied to the seeds */
    int32_t flags;                 /* FGL_SAMPLE_REPLACE | FGL_MAP_ARRIVAL_ORDER */
    int32_t n_teams;               /* mini-batches in flight at once (0 = library default) */
    int64_t table_slots_hint;      /* 0 = size each team's table for the worst case; else an expected
                                      number of slots (rounded up to a power of two).  A table that fills up
                                      makes the launch report FGL_ERR_PROBE. */
    uint64_t rng_seed;
    uint64_t rng_ctr;              /* mini-batch b, hop h draws with counter rng_ctr + b * 8 + h */
    const int32_t* seeds;          /* [n_batches][seed_stride] */
    int64_t seed_stride;
    const int32_t* seed_counts;    /* int32[n_batches], each <= seed_stride */
    int32_t* nodes;                /* out [n_batches][nodes_stride]: unique global ids, seeds first; the
                                      first counts[b][h] entries are the destination nodes of hop h */
    int64_t nodes_stride;
    int32_t* counts;               /* out [n_batches][FGL_COUNTS_STRIDE] */
    int32_t* block_indptr[FGL_MAX_HOPS];     /* out, hop h: [n_batches][block_indptr_stride[h]] */
    int64_t block_indptr_stride[FGL_MAX_HOPS];
    int32_t* block_src[FGL_MAX_HOPS];        /* out, hop h: [n_batches][block_src_stride[h]] local ids */
    int64_t block_src_stride[FGL_MAX_HOPS];
} fgl_fused_args;

/* Capacities a caller must allocate: cap_nodes[h] bounds counts[b][h] (h = 0 .. n_hops), the hop-h
 * block needs cap_nodes[h] + 1 indptr entries and cap_nodes[h] * fanout[h] source entries. */
int fgl_fused_capacity(int64_t n_nodes, int32_t max_seeds, int32_t n_hops, const int32_t* fanout,
                       int64_t* cap_nodes /* n_hops + 1 */);
int fgl_sample_map_fused(fgl_ws* ws, const fgl_fused_args* args, void* stream);

/* Histogram of an id array; replaces cal_deg_cuda (utilis.cu:60-79; binding aggregate_acc.cpp:522-529).
 * deg[0 .. n_nodes) is zeroed and then counts the occurrences of each id. */
int fgl_cal_deg(const int32_t* ids, int64_t n_ids, int32_t* deg, int32_t n_nodes, void* stream);

/* Stages one mini-batch into fixed buffers: up to FGL_MAX_SEGMENTS device-to-device copies (sizes and
 * addresses multiples of 4 bytes) and up to FGL_MAX_SEGMENTS int32 words written to words_dst, in one kernel
 * launch.  No counterpart in the reference; it feeds the static inputs of a captured CUDA graph (block CSR
 * arrays, first-layer rows, row counts) without one cudaMemcpyAsync per piece. */
#define FGL_MAX_SEGMENTS 8
typedef struct fgl_segment {
    void* dst;
    const void* src;
    int64_t bytes;
} fgl_segment;
int fgl_stage_segments(const fgl_segment* segs, int32_t n_segs, int32_t* words_dst, const int32_t* words,
                       int32_t n_words, void* stream);

/* Pairwise overlap of the node lists of a window of mini-batches, on the device: overlap[i * n_batches + j] =
 * |nodes_i & nodes_j| (the diagonal holds the list lengths).  This is the quantity behind Match-Reorder's match
 * degree (match_reorder.reorder, utilis.py:41-48), which the reference derives from one N-sized boolean mask per
 * mini-batch (utilis.py:27-28).  nodes is int32 [n_batches][nodes_stride] as fgl_sample_map_fused leaves it, the
 * list of batch b being its first counts[b * counts_stride] entries (ids distinct within a list); n_batches <= 32.
 * mask is caller-owned scratch of n_nodes 32-bit words that must be zero on entry and is zero again on return. */
int fgl_window_overlap(const int32_t* nodes, int64_t nodes_stride, const int32_t* counts, int64_t counts_stride,
                       int32_t n_batches, int64_t n_nodes, uint32_t* mask, int32_t* overlap, void* stream);

/* Exclusive scan with the total appended; replaces exclusive_sum_cuda (utilis.cu:17-41; binding
 * aggregate_acc.cpp:514-520).  out has n + 1 entries. */
int fgl_exclusive_sum(fgl_ws* ws, const int32_t* in, int64_t n, int32_t* out, void* stream);

/* The same scan for callers that cannot allocate device memory (a plugin under a framework allocator's
 * fixed budget, a process whose HBM is fully handed out to other pools, a loop that cannot take
 * cudaMalloc's device synchronisation).  No counterpart in the reference, which allocates scratch in every
 * call.  The scratch (one barrier counter and one partial sum per CTA, about 4.5 KB) lives in a __device__
 * array of the library, held by every GPU that loads it; the call takes no workspace and calls no allocating routine.  n may not exceed
 * FGL_NOALLOC_MAX_N (else FGL_ERR_CAPACITY).  The first call on a device looks up the array's device
 * address (cudaGetSymbolAddress) and should come before any stream capture.  All calls on a device share
 * the array: calls whose kernels overlap on the GPU (different streams) race.  Launches on the current
 * device. */
#define FGL_NOALLOC_MAX_N (1LL << 27)
int fgl_exclusive_sum_noalloc(const int32_t* in, int64_t n, int32_t* out, void* stream);
/* How such a caller learns that a scan's bounded barrier gave up (its output is then incomplete): enqueues, on the
 * stream, a copy of the array's status word to host_dst (one int32 of host memory; pinned if the copy is to stay
 * asynchronous) followed by clearing the word -- FGL_OK, or FGL_ERR_TIMEOUT if any scan since the last such call
 * timed out.  Allocates nothing either; read *host_dst after synchronising the stream. */
int fgl_exclusive_sum_noalloc_status(int32_t* host_dst, void* stream);

/* Aggregation forward; replaces the gather kernels K8 / K10 of the reference
 * (computation_aware_forward_gcn_cuda_kernel aggregate_acc_kernel.cu:271-331 and
 * computation_aware_forward_gin_cuda_kernel :376-427).  out[d, 0..dim) = sum over e in
 * [indptr[d], indptr[d+1]) of w * x[row(src[e]), 0..dim), with w by mode and row(i) = row_map[i] if
 * row_map is not NULL (aggregation straight from a feature table by global id) else i.  src_deg /
 * dst_deg are only read in FGL_AGG_SYMNORM.
 * Bounds: x has n_rows rows and row_map (if any) n_map entries.  The reference dereferences whatever id the
 * block holds (:316-324); here an id outside [0, n_map) or a row outside [0, n_rows) is never dereferenced: the
 * edge contributes nothing (a gathered row or a row's own copy becomes zeros) and FGL_ERR_BOUNDS is recorded in
 * the status word of ws (fgl_ws_check).  ws may be NULL: bad ids are then skipped silently.  This holds for every
 * aggregation entry point below.
 * n_dst_dev (may be NULL) points at the real row count in device memory; n_dst is then the padded count the
 * launch is sized for (rows beyond the real count are zero-filled), which lets a captured CUDA graph be
 * replayed on blocks of different sizes. */
int fgl_agg_fwd(fgl_ws* ws, int32_t mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg,
                const int32_t* dst_deg, const int32_t* row_map, int64_t n_map, const float* x, int64_t n_rows,
                int64_t ldx, int32_t dim, int32_t n_dst, int32_t flags, float* out, int64_t ldo,
                const int32_t* n_dst_dev, void* stream);

/* fgl_agg_fwd over a feature table that is row-sharded across GPUs: shards (device array of n pointers, each a
 * table of the same leading dimension, mapped into this GPU's address space -- its own HBM or a peer's over
 * NVLink) replaces x (x may then be NULL); global row r is shards[r / rows_per_shard][r % rows_per_shard].
 * Rows are fetched with plain 128-bit peer loads, each warp its own rows: no collective, no TMA multicast.
 * No counterpart in the reference, which keeps features on the host (train_fastgl.py:233). */
int fgl_agg_fwd_sharded(fgl_ws* ws, int32_t mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg,
                        const int32_t* dst_deg, const int32_t* row_map, int64_t n_map, const float* x,
                        const float* const* shards, int64_t rows_per_shard, int64_t n_rows, int64_t ldx, int32_t dim,
                        int32_t n_dst, int32_t flags, float* out, int64_t ldo, const int32_t* n_dst_dev, void* stream);

/* Edge-weighted multi-head aggregation; replaces computation_aware_forward_gat_cuda /
 * computation_aware_backward_gat_cuda (aggregate_acc_kernel.cu:789-979; bindings aggregate_acc.cpp
 * forward_gat / backward_gat).  edge_w is float32 [n_edges][n_heads] (the attention coefficients after the
 * edge softmax), head h owns columns [h * dim / n_heads, (h + 1) * dim / n_heads).
 * Forward: out[d, f] = sum over row d's edges e of edge_w[e, head(f)] * x[src[e], f]; a row without in-edges
 * copies x[d] when FGL_AGG_ZERO_DEG_PASSTHROUGH is set (:870-872).  Backward: dx is zero-filled, then
 * dx[src[e], f] += edge_w[e, head(f)] * dy[d, f]; like the reference, no gradient flows to edge_w. */
int fgl_agg_edge_fwd(fgl_ws* ws, const int32_t* indptr, const int32_t* src, const float* edge_w, int32_t n_heads,
                     const float* x, int32_t n_src, int64_t ldx, int32_t dim, int32_t n_dst, int32_t flags, float* out,
                     int64_t ldo, void* stream);
int fgl_agg_edge_bwd(fgl_ws* ws, const int32_t* indptr, const int32_t* src, const float* edge_w, int32_t n_heads,
                     const float* dy, int64_t ldy, int32_t dim, int32_t n_dst, int32_t n_src, float* dx, int64_t ldx,
                     void* stream);

/* Gradient of the attention coefficients, which the reference does not compute (MA_Function_GAT.backward returns
 * None for edge_data, GraphConv.py:227): dw[e, h] = sum over head h's columns f of dy[d, f] * x[src[e], f] for
 * every edge e of row d.  dw is float32 [n_edges][n_heads] and is zero-filled first. */
int fgl_agg_edge_wgrad(fgl_ws* ws, const int32_t* indptr, const int32_t* src, int32_t n_heads, const float* x,
                       int32_t n_src, int64_t ldx, const float* dy, int64_t ldy, int32_t dim, int32_t n_dst,
                       int64_t n_edges, float* dw, void* stream);

/* Row gather out[i, :] = table[ids[i], :] from a single table (shards = NULL) or a row-sharded one (table may
 * be NULL) of n_rows rows, as above; an id outside [0, n_rows) gives a row of zeros and FGL_ERR_BOUNDS.  Replaces the CPU index_select + host-to-device copy of load_subtensors
 * (train_fastgl.py:161-184) and the MatchServer cache look-ups (MatchReorderServer.py:79-110). */
int fgl_gather_rows(fgl_ws* ws, const float* table, const float* const* shards, int64_t rows_per_shard, int64_t n_rows,
                    int64_t ld, int32_t dim, const int32_t* ids, int64_t n_ids, float* out, int64_t ldo, void* stream);

/* Forward aggregation (FGL_AGG_SUM or FGL_AGG_MEAN) of one layer for a whole window of mini-batches in one
 * launch, laid out as fgl_sample_map_fused leaves them: batch b's block is indptr + b * indptr_stride,
 * src + b * src_stride, its row map (may be NULL) row_map + b * row_map_stride.  out_row_off (device,
 * n_batches + 1 entries) is the exclusive prefix sum of the batches' destination-row counts followed by the
 * total (= total_rows); batch b's row d lands at out[(out_row_off[b] + d) * ldo].  If self_out is not
 * NULL, the row's own input row x[row(d)] is copied to self_out[(out_row_off[b] + d) * ld_self] as well
 * (the "self" operand of a GraphSAGE layer).  Rows are processed in batch-major order so that a batch's
 * re-read source rows stay in L2.  Used for the first layer, which reads only the feature table and does
 * not depend on the weights; the reference runs K10 once per mini-batch (GraphConv.py:109) after a CPU
 * gather of the input rows (train_fastgl.py:161-184).  x / shards / rows_per_shard as in
 * fgl_agg_fwd_sharded. */
int fgl_agg_fwd_window(fgl_ws* ws, int32_t mode, int32_t n_batches, const int32_t* indptr, int64_t indptr_stride,
                       const int32_t* src, int64_t src_stride, const int32_t* row_map, int64_t row_map_stride,
                       const int64_t* out_row_off, int64_t total_rows, const float* x, const float* const* shards,
                       int64_t rows_per_shard, int64_t n_rows, int64_t ldx, int32_t dim, int32_t flags, float* out,
                       int64_t ldo, float* self_out, int64_t ld_self, void* stream);

/* Aggregation backward; replaces the scatter kernels K9 / K11
 * (computation_aware_backward_gcn_cuda_kernel aggregate_acc_kernel.cu:468-517 and
 * computation_aware_backward_gin_cuda_kernel :555-596).  dx[0 .. n_src) is zeroed, then
 * dx[src[e], :] += w * dy[d, :] for every edge e of row d.  Rows without in-edges contribute nothing
 * (as the reference, :498-500, :580-582).  n_dst_dev as in fgl_agg_fwd (n_src is never read from the
 * device: dx is zero-filled over all n_src rows). */
int fgl_agg_bwd(fgl_ws* ws, int32_t mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg,
                const int32_t* dst_deg, const float* dy, int64_t ldy, int32_t dim, int32_t n_dst,
                int32_t n_src, float* dx, int64_t ldx, const int32_t* n_dst_dev, void* stream);

/* fgl_agg_bwd for a layer that also feeds each destination's own row forward (GraphSAGE: [h_dst | aggregate]):
 * dx starts as dy_self in its first n_dst rows (the destinations are the first n_dst sources) and zero below,
 * then receives the scattered dy as above -- one pass instead of a zero-fill, a scatter, a padded copy and an
 * add.  dy_self is float32 [n_dst][dim] with leading dimension ld_self; n_dst <= n_src.  With n_dst_dev the
 * rows of dy_self at or beyond the real count are ignored (dx is zero there), whatever they hold.  No counterpart in the
 * reference, whose models have no self term (GraphConv.py:86-99). */
int fgl_agg_bwd_self(fgl_ws* ws, int32_t mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg,
                     const int32_t* dst_deg, const float* dy, int64_t ldy, const float* dy_self, int64_t ld_self,
                     int32_t dim, int32_t n_dst, int32_t n_src, float* dx, int64_t ldx, const int32_t* n_dst_dev,
                     void* stream);

/* Aggregation backward as a gather, deterministic: the same result as fgl_agg_bwd / fgl_agg_bwd_self (the scatters
 * K9 / K11 of the reference, aggregate_acc_kernel.cu:468-517, :555-596, which add with atomics in arbitrary order), but
 * every row dx[s] is produced by one warp -- or, for a source with more than 32 edges in the block, one CTA -- that
 * adds the rows dy[d] of the edges (d, s) in ascending order of d.  Two runs give the same bits; dx needs no
 * initialisation (rows without edges become zero, or dy_self[s]); dy_self may be NULL.
 *
 * fgl_block_transpose builds the per-source lists once per block: t_indptr (n_src + 1 offsets), t_dst (the edges'
 * destination rows grouped by source, t_cap >= number of edges), hubs (n_src + 1 words: the number of sources with
 * more than 32 edges, then their ids).  work is scratch of 2 * n_src words.  A source id outside [0, n_src) records
 * FGL_ERR_BOUNDS and is skipped.  n_dst_dev as in fgl_agg_fwd. */
int fgl_block_transpose(fgl_ws* ws, const int32_t* indptr, const int32_t* src, int32_t n_dst, int32_t n_src,
                        int32_t* t_indptr, int32_t* t_dst, int64_t t_cap, int32_t* hubs, int32_t* work,
                        const int32_t* n_dst_dev, void* stream);
int fgl_agg_bwd_gather(fgl_ws* ws, int32_t mode, const int32_t* indptr, const int32_t* t_indptr, const int32_t* t_dst,
                       const int32_t* hubs, const int32_t* src_deg, const int32_t* dst_deg, const float* dy, int64_t ldy,
                       const float* dy_self, int64_t ld_self, int32_t dim, int32_t n_dst, int32_t n_src, float* dx,
                       int64_t ldx, const int32_t* n_dst_dev, void* stream);

/* ---- Element-wise kernels of the training step around the aggregation path -----------------------------
 * None of these has a counterpart among the reference's CUDA operators: the reference leaves them to PyTorch,
 * op by op (model code GraphConv.py:86-99,182-195; loss and optimizer train_fastgl.py:366-372).  They exist so
 * that a whole training step can be a short, capturable sequence of launches. */

/* y[r, c] = dropout(relu(y[r, c] + bias[c])) in place over n_rows x dim (leading dimension ld).  bias may be NULL;
 * FGL_EW_RELU in flags applies the ReLU; p_drop in [0, 1) (0 = no dropout; survivors are scaled by 1 / (1 - p)).
 * Element e = r * dim + c is dropped when word (e & 3) of the Philox4x32-10 block with key rng_seed and counter
 * (lo32(e >> 2), hi32(e >> 2), lo32(ctr), hi32(ctr)) is below p_drop * 2^32, where ctr = rng_ctr plus, when
 * rng_ctr_dev is not NULL, the unsigned value rng_ctr_dev[0] read on the device (a per-step counter that lets a
 * captured launch draw a fresh mask on every replay).  When copy_out is not NULL the first n_copy_rows result
 * rows are also stored to copy_out (leading dimension ld_copy): the self operand of the next GraphSAGE layer. */
int fgl_bias_relu_dropout(float* y, int64_t ld, int64_t n_rows, int32_t dim, const float* bias, float p_drop,
                          uint64_t rng_seed, uint64_t rng_ctr, const int32_t* rng_ctr_dev, int32_t flags, float* copy_out,
                          int64_t ld_copy, int64_t n_copy_rows, void* stream);

/* Backward of fgl_bias_relu_dropout: with FGL_EW_RELU, dy[r, c] becomes dy[r, c] / (1 - p_drop) where the
 * forward output out[r, c] is positive and 0 elsewhere (an element is positive exactly when it passed both the
 * ReLU and the dropout); without the flag dy is left as it is.  dbias (may be NULL; dim <= 2048) is incremented
 * by the column sums of the resulting dy: the caller zeroes it. */
int fgl_relu_dropout_bwd(float* dy, int64_t ldy, const float* out, int64_t ldo, int64_t n_rows, int32_t dim, float p_drop,
                         float* dbias, int32_t flags, void* stream);

/* fgl_relu_dropout_bwd whose result is not written back over dy but as error-compensated TF32 operands (see
 * fgl_split_tf32): split3[r, c] = hi, split3[r, block_stride + c] = lo, split3[r, 2 * block_stride + c] = hi of
 * dz[r, c]; split3 has leading dimension ld3 >= 2 * block_stride + dim.  dy is only read. */
int fgl_relu_dropout_bwd_split(const float* dy, int64_t ldy, const float* out, int64_t ldo, int64_t n_rows, int32_t dim,
                               float p_drop, float* dbias, int32_t flags, float* split3, int64_t ld3, int64_t block_stride,
                               void* stream);

/* Mean softmax cross-entropy over the first n_valid rows and its gradient.  The label of row r is
 * labels[label_ids ? label_ids[r] : r] (labels: int64[n_labels], values in [0, n_classes); an index or a label
 * outside its range records FGL_ERR_BOUNDS in the workspace's status word and the row contributes nothing).  n_valid is read from n_valid_dev[0] when that is not NULL.
 * loss[0] = mean over valid rows of logsumexp(z_r) - z_r[label]; dlogits[r, :] = (softmax(z_r) - onehot) / n_valid
 * for valid rows and 0 for the others.  row_loss is caller-owned scratch of n_rows floats (it receives the per-row
 * losses, which are then summed in a fixed order: the loss is reproducible).  The workspace only lends its
 * status word. */
int fgl_softmax_xent(fgl_ws* ws, const float* logits, int64_t ld, const int64_t* labels, const int32_t* label_ids,
                     int64_t n_labels, int32_t n_rows, int32_t n_classes, const int32_t* n_valid_dev, int32_t n_valid,
                     float* loss, float* dlogits, int64_t ldd, float* row_loss, void* stream);

/* The output layer and its loss in one pass, for n_classes <= 128: logits = x W + bias (x float32[n_rows][k], W
 * float32[k][n_classes] row-major, bias may be NULL), then exactly what fgl_softmax_xent computes from those
 * logits (same label lookup, masking, loss and dlogits).  dbias (may be NULL) is incremented by the column sums of
 * dlogits (the caller zeroes it); logits_out (may be NULL) receives the logits of every row. */
int fgl_linear_softmax_xent(fgl_ws* ws, const float* x, int64_t ldx, int32_t k, const float* w, int64_t ldw, const float* bias,
                            const int64_t* labels, const int32_t* label_ids, int64_t n_labels, int32_t n_rows,
                            int32_t n_classes, const int32_t* n_valid_dev, int32_t n_valid, float* loss, float* dlogits,
                            int64_t ldd, float* dbias, float* logits_out, int64_t ldl, float* row_loss, void* stream);

/* One Adam step with L2 weight decay over flat fp32 buffers of n elements (16-byte aligned), with the arithmetic
 * of torch.optim.Adam: g += wd * p; m = b1 m + (1 - b1) g; v = b2 v + (1 - b2) g^2;
 * p -= lr / (1 - b1^t) * m / (sqrt(v) / sqrt(1 - b2^t) + eps), t = step_dev[0] + 1.  step_dev is two int32 words
 * in device memory, zero before the first step: [0] counts completed steps and is advanced by the launch itself
 * (so a captured launch advances on every replay), [1] is scratch that is zero between launches. */
int fgl_adam_step(float* param, const float* grad, float* exp_avg, float* exp_avg_sq, int64_t n, float lr, float beta1,
                  float beta2, float eps, float weight_decay, int32_t* step_dev, void* stream);

/* Error-compensated operands for tensor-core products of fp32 matrices: hi = x rounded to TF32 (10-bit mantissa,
 * round to nearest), lo = (x - hi) rounded to TF32; both are stored as fp32 words whose low 13 mantissa bits are
 * zero, so a TF32 GEMM reads them without loss.  A.B ~= Ahi.Bhi + Alo.Bhi + Ahi.Blo with fp32 accumulation has
 * fp32-level error (the dropped lo.lo term is 2^-22 relative).  Each part can be written to several destinations
 * -- row or column blocks of wider matrices -- so that the sum of the three products is one GEMM over a three
 * times longer inner dimension: [Ahi | Alo | Ahi] . [Bhi ; Bhi ; Blo].  The reference leaves its dense products
 * to torch::mm (aggregate_acc_kernel.cu:237,368), which on its pinned PyTorch 1.10 ran them in single-pass TF32.
 * x: rows x cols with leading dimension ldx; dst[q] (q < n_dst <= 8): rows x cols with leading dimension
 * ld_dst[q], receiving lo if lo_part[q] != 0, else hi.  dst, ld_dst and lo_part are host arrays.  No destination
 * may overlap x. */
int fgl_split_tf32(const float* x, int64_t rows, int64_t cols, int64_t ldx, int n_dst, float* const* dst, const int64_t* ld_dst,
                   const int32_t* lo_part, void* stream);

/* out[r, c] = sum over s < n_slabs, a < n_a, b < n_b of part[s][a * rows + r][b * block_stride + c], part being
 * n_slabs matrices of n_a * rows rows with leading dimension ld_part, slab_stride floats apart.  Folds the 2 x 2
 * block product [X_hi | X_lo]^T [dZ_hi | dZ_lo] of split operands (fgl_split_tf32) and its split-K slabs into the
 * rows x cols weight gradient, in float32 (a product with a vector of ones would round the partial sums to TF32). */
int fgl_fold_blocks(const float* part, int32_t n_slabs, int32_t n_a, int32_t n_b, int32_t rows, int32_t cols, int32_t block_stride,
                    int64_t ld_part, int64_t slab_stride, float* out, int64_t ldo, void* stream);

/* ---- Data-parallel gradient exchange -----------------------------------------------------------------------
 * The reference trains its replicas without synchronising gradients at all (train_fastgl.py:204-212,404-405);
 * a data-parallel run that is to converge like a single-GPU run needs the average of the ranks' gradients before
 * the optimizer step.  fgl_allreduce_adam does both in ONE launch per step, without a library collective: every
 * rank pushes its flat gradient into the receive buffers of the other ranks with plain peer stores over
 * NVLink, raises a flag per 8 KB chunk, waits (bounded) for the other ranks' flags, adds the contributions in rank
 * order (identical on every rank, so the replicas stay bit-identical), scales by 1 / world, writes the average
 * back to grad and applies fgl_adam_step's arithmetic to param / exp_avg / exp_avg_sq.
 *
 * peers describes the buffers as they are mapped into THIS process (CUDA IPC or any other peer mapping):
 * recv[q] is rank q's receive buffer, float[2][world][n_pad], and flags[q] rank q's flag array,
 * uint32[2][world][n_chunks], both zero before the first call; n_chunks = fgl_peer_sync_chunks(n) and
 * n_pad >= n_chunks * 2048.  step_dev is three int32 words, zero before the first step: [0] completed optimizer
 * steps, [1] scratch, [2] completed exchanges; the launch advances them itself, so it can be captured in a CUDA
 * graph and replayed.  Every rank must issue the same sequence of calls.  With world = 1 nothing is exchanged.
 * A wait gives up after spin_limit polls (about a microsecond each): the chunk's parameters are then left as they
 * were and FGL_ERR_TIMEOUT is recorded in the workspace's status word.  n is a multiple of 4, buffers 16-byte
 * aligned. */
#define FGL_MAX_PEERS 8
typedef struct fgl_peer_sync {
    int32_t rank, world;
    float* recv[FGL_MAX_PEERS];
    uint32_t* flags[FGL_MAX_PEERS];
    int64_t n_pad;
    int32_t n_chunks;
} fgl_peer_sync;
int fgl_sizeof_peer_sync(void);
int64_t fgl_peer_sync_chunks(int64_t n);
int fgl_allreduce_adam(fgl_ws* ws, const fgl_peer_sync* peers, float* param, float* grad, float* exp_avg,
                       float* exp_avg_sq, int64_t n, float lr, float beta1, float beta2, float eps, float weight_decay,
                       int32_t* step_dev, int64_t spin_limit, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FASTGL_B200_H_ */
