// Neighbour sampling and the Fused-Map id mapping for sm_100a.
//
// One persistent, cooperatively launched kernel walks every hop of every mini-batch it is given.  Its
// CTAs are split into teams; a team owns one mini-batch at a time and one slice of the hashtable that is
// small enough to stay in the 126 MB L2, and synchronises with a team-local barrier, so that several
// mini-batches are in flight and one team's barrier latency is covered by the others' memory traffic.
//
// Per hop, for the current node list (the seeds of the hop), in the fused kernel:
//   A  count     k_s = min(deg, fanout) per seed from the degrees cached when the node joined the list (coalesced),
//                one partial sum per CTA
//   B  sample    block-CSR offsets by a two-level scan; each seed is served by a group of 8/16/32 lanes that choose
//                the picks (Philox4x32-10; Floyd's algorithm for a k-subset, run by the group in registers), read the
//                picked sources and insert them into the open-addressing table (64-bit slots {key, value}, atomicCAS
//                to claim, atomicMin of the edge number to find the first occurrence).  A thread that claims a slot or
//                lowers its edge number marks its edge "possibly first" and moves one unit of the per-CTA count of
//                first occurrences from the displaced edge's CTA to its own, so no counting pass is needed
//   D  rank      scan over the possibly-first edges that still hold their slot -> local id, publish it in the slot,
//                append the node (and its adjacency offset and degree, for the next hop) to the list
//   E  relabel   replace the slot position kept in the remaining edge entries by the local id
// With FGL_MAP_ARRIVAL_ORDER the claiming thread takes the next id from a warp-aggregated counter in phase B and
// phase D is skipped.  The drop-in kernels (fgl_sample: phases A + B without a table; fgl_map: explicit edges) keep
// a counting pass (C) between B and D.
//
// Replaces sample_node_cuda (sample.cu:102-203), transfer_edge_id_cuda (id_map.cu:386-493) and the
// hashtable of id_map.cu:26-255 / cuda_hashtable.cuh.
#include <cooperative_groups.h>

#include <algorithm>
#include <cstring>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace fgl {

#ifndef FGL_SM_THREADS
#define FGL_SM_THREADS 512
#endif
constexpr int kThreads = FGL_SM_THREADS;
constexpr int kMinCtas = 1024 / FGL_SM_THREADS;
constexpr int kWarps = kThreads / 32;
constexpr unsigned long long kEmpty = ~0ULL;
constexpr uint32_t kPending = 0x80000000u;

enum { MODE_FUSED = 0, MODE_SAMPLE = 1, MODE_MAP = 2 };

struct KParams {
    // graph
    const void* indptr;
    const int32_t* indices;
    int64_t n_nodes;
    // batch geometry
    int32_t n_batches, n_hops;
    int32_t fanout[FGL_MAX_HOPS];
    int32_t flags;
    int32_t n_teams, team_size;
    uint64_t rng_seed, rng_ctr;
    const int32_t* seeds;
    int64_t seed_stride;
    const int32_t* seed_counts;  // device; if NULL every batch has n_seeds_host seeds
    int32_t n_seeds_host;
    int32_t* nodes;
    int64_t nodes_stride;
    int32_t* counts;
    int32_t* blk_indptr[FGL_MAX_HOPS];
    int64_t blk_indptr_stride[FGL_MAX_HOPS];
    int32_t* blk_src[FGL_MAX_HOPS];
    int64_t blk_src_stride[FGL_MAX_HOPS];
    int32_t* out_dst;  // MODE_SAMPLE: global seed id per edge (may be NULL)
    // MODE_MAP: explicit edges
    int32_t* map_src;
    int32_t* map_dst;
    int64_t map_edges;
    // workspace
    unsigned long long* table;
    int64_t table_slots;  // per team, power of two
    int32_t table_shift;  // 32 - log2(table_slots)
    unsigned long long* barriers;  // one per team, 16 words apart
    int32_t* team_sums;            // [n_teams][team_size]: per-CTA edge counts of the hop
    int32_t* team_cnt;             // [n_teams][team_size]: per-CTA counts of first occurrences (fused kernel)
    long long* node_start;         // [n_teams][deg_stride]: adjacency offset of every node that can still be a seed
    int32_t* node_deg;             // [n_teams][deg_stride]: and its degree
    int64_t deg_stride;
    int32_t* status;               // [0] first error, [1] abort flag
};

// ----------------------------------------------------------------------------------------------
// hashtable: 64-bit slots, key in the high word; low word = local id (bit 31 clear) or, while the
// key's id is not assigned yet, kPending | (smallest edge number that carries the key)
// ----------------------------------------------------------------------------------------------
struct Table {
    unsigned long long* slots;
    uint32_t mask;
    int shift;
};

__device__ __forceinline__ uint32_t hash_pos(const Table& t, uint32_t key) { return (key * 0x9E3779B1u) >> t.shift; }

__device__ __forceinline__ unsigned long long ld_slot(const unsigned long long* p) {
    return *(const volatile unsigned long long*)p;
}

// A picked neighbour id is read once and never again: a hub's list has thousands of entries and a pick touches one
// 32-byte sector of it.  The load tells the L2 to evict that line first and keeps it out of L1, so the picks do not
// push the teams' tables and the next phase's entries out of the L2 (measured: 7 % off the launch; marking the table
// accesses evict-last on top of it bought nothing and slowed the aggregation kernel that shares the L2).
__device__ __forceinline__ int ld_adjacency(const int32_t* p) {
    int v;
    uint64_t policy;
    asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(policy));
    return v;
}

// A probe sequence gives up after kProbeLimit slots (or the whole table, if smaller): at the load factors the
// tables are sized for (<= 2/3) clusters are a few slots long, so only a table that is too small for its
// mini-batch gets there.  The failure is recorded and the launch is told to stop at its next team barrier, so an
// undersized table costs milliseconds, not a scan of the table per key.
constexpr uint32_t kProbeLimit = 1u << 13;

__device__ __forceinline__ uint32_t probe_limit(const Table& t) { return t.mask < kProbeLimit ? t.mask : kProbeLimit; }

__device__ __forceinline__ void probe_failed(int32_t* status) {
    set_status(status, FGL_ERR_PROBE);
    atomicExch(status + 1, 1);
}

// Seed i gets local id i; of two equal seeds the later position wins, as a sequential run of
// id_map.cu:259-287 leaves it.
// Returns the slot position, or -1 when the table is full.
__device__ __forceinline__ int table_insert_seed(const Table& t, uint32_t key, uint32_t local, int32_t* status) {
    const unsigned long long mine = ((unsigned long long)key << 32) | local;
    uint32_t pos = hash_pos(t, key);
    for (uint32_t probe = 0; probe <= probe_limit(t); ++probe) {
        unsigned long long cur = ld_slot(t.slots + pos);
        if (cur == kEmpty) {
            cur = atomicCAS(t.slots + pos, kEmpty, mine);
            if (cur == kEmpty) return (int)pos;
        }
        if ((uint32_t)(cur >> 32) == key) {
            atomicMax(t.slots + pos, mine);
            return (int)pos;
        }
        pos = (pos + 1) & t.mask;
    }
    probe_failed(status);
    return -1;
}

// Returns the local id (>= 0) if the key already has one, else ~pos of its slot (< 0).  created is set
// for the thread whose atomicCAS claimed the slot.
template <bool ARRIVAL>
__device__ __forceinline__ int table_insert_from(const Table& t, uint32_t key, uint32_t edge, uint32_t pos,
                                                 int32_t* status, bool& created) {
    created = false;
    const unsigned long long mine = ((unsigned long long)key << 32) | (ARRIVAL ? kPending : (kPending | edge));
    for (uint32_t probe = 0; probe <= probe_limit(t); ++probe) {
        unsigned long long cur = ld_slot(t.slots + pos);
        if (cur == kEmpty) {
            cur = atomicCAS(t.slots + pos, kEmpty, mine);
            if (cur == kEmpty) {
                created = true;
                return ~(int)pos;
            }
        }
        if ((uint32_t)(cur >> 32) == key) {
            const uint32_t lo = (uint32_t)cur;
            if (!(lo & kPending)) return (int)lo;
            if (!ARRIVAL && lo > (kPending | edge)) atomicMin(t.slots + pos, mine);
            return ~(int)pos;
        }
        pos = (pos + 1) & t.mask;
    }
    probe_failed(status);
    return 0;
}

template <bool ARRIVAL>
__device__ __forceinline__ int table_insert(const Table& t, uint32_t key, uint32_t edge, int32_t* status,
                                            bool& created) {
    return table_insert_from<ARRIVAL>(t, key, edge, hash_pos(t, key), status, created);
}

// Lowers the edge number kept in a pending slot to `edge` if that is smaller.  Returns the edge number that lost
// its place as the key's first occurrence, or -1 if nothing changed.
__device__ __forceinline__ int table_lower_edge(const Table& t, uint32_t pos, uint32_t key, uint32_t edge) {
    const unsigned long long mine = ((unsigned long long)key << 32) | (kPending | edge);
    const unsigned long long old = atomicMin(t.slots + pos, mine);
    const uint32_t old_lo = (uint32_t)old;
    return ((old_lo & kPending) && old_lo > (kPending | edge)) ? (int)(old_lo & ~kPending) : -1;
}

// table_insert_from for the fused kernel's first-occurrence order: also reports the edge this insert displaced as the
// key's first occurrence (-1: none).  created or displaced >= 0 means "edge may be the key's first occurrence".
__device__ __forceinline__ int table_insert_track(const Table& t, uint32_t key, uint32_t edge, uint32_t pos,
                                                  int32_t* status, bool& created, int& displaced) {
    created = false;
    displaced = -1;
    const unsigned long long mine = ((unsigned long long)key << 32) | (kPending | edge);
    for (uint32_t probe = 0; probe <= probe_limit(t); ++probe) {
        unsigned long long cur = ld_slot(t.slots + pos);
        if (cur == kEmpty) {
            cur = atomicCAS(t.slots + pos, kEmpty, mine);
            if (cur == kEmpty) {
                created = true;
                return ~(int)pos;
            }
        }
        if ((uint32_t)(cur >> 32) == key) {
            const uint32_t lo = (uint32_t)cur;
            if (!(lo & kPending)) return (int)lo;
            if (lo > (kPending | edge)) displaced = table_lower_edge(t, pos, key, edge);
            return ~(int)pos;
        }
        pos = (pos + 1) & t.mask;
    }
    probe_failed(status);
    return 0;
}

// Value of a key that must be present (a seed); missing keys report FGL_ERR_BOUNDS and map to 0.
__device__ __forceinline__ int table_lookup(const Table& t, uint32_t key, int32_t* status) {
    uint32_t pos = hash_pos(t, key);
    for (uint32_t probe = 0; probe <= probe_limit(t); ++probe) {
        const unsigned long long cur = ld_slot(t.slots + pos);
        if (cur == kEmpty) break;
        if ((uint32_t)(cur >> 32) == key) return (int)((uint32_t)cur & ~kPending);
        pos = (pos + 1) & t.mask;
    }
    set_status(status, FGL_ERR_BOUNDS);
    return 0;
}

// ----------------------------------------------------------------------------------------------
// per-hop state
// ----------------------------------------------------------------------------------------------
struct Hop {
    int32_t* nodes;        // this mini-batch's unique list
    int64_t nodes_cap;
    int32_t* counts;       // this mini-batch's counts row
    int32_t* blk_indptr;   // may be NULL (MODE_SAMPLE without CSR output)
    int32_t* blk_src;      // edge array: global ids (MODE_SAMPLE) or local ids / pending entries
    int32_t* out_dst;      // MODE_SAMPLE only
    long long* node_start; // fused: adjacency offset and degree of the nodes that can still become seeds
    int32_t* node_deg;
    int64_t deg_cap;
    int hop, fanout, n_seeds;
    bool last_hop;
    uint64_t ctr;
};

constexpr int kMaxTeam = 512;  // CTAs per team (a cooperative grid of 512-thread CTAs has at most a few hundred)

struct Smem {
    int scan[40];
    int flag;
    int v[kThreads];
    long long start[kThreads];
    int deg[kThreads];
    int off[kThreads];
    int prefix[kMaxTeam + 1];  // fused: first edge of every CTA of the team (the owner of an edge number)
};

// Fused kernel, first-occurrence order: an edge entry is a local id (>= 0) or, while the id is pending,
// ~(slot | kTentative if the edge may be the first occurrence of its key).  Slots are below 2^29.
constexpr int kTentative = 1 << 29;
constexpr int kSlotMask = kTentative - 1;

__device__ __forceinline__ void chunk_of(int n, int rank, int size, int& lo, int& hi) {
    const int per = (n + size - 1) / size;
    lo = min(n, rank * per);
    hi = min(n, lo + per);
}

template <typename PtrT>
__device__ __forceinline__ void load_adj(const KParams& p, int v, long long& start, int& deg) {
    const PtrT* ptr = (const PtrT*)p.indptr;
    if (v < 0 || (int64_t)v >= p.n_nodes) {
        set_status(p.status, FGL_ERR_BOUNDS);
        start = 0;
        deg = 0;
        return;
    }
    const long long a = (long long)ptr[v], b = (long long)ptr[v + 1];
    start = a;
    const long long d = b - a;
    deg = d < 0 ? 0 : (d > 0x7fffffffLL ? 0x7fffffff : (int)d);
}

// The CTA of the team whose edge range holds edge number e (sm.prefix is the exclusive scan of the CTAs' edge counts).
__device__ __forceinline__ int edge_owner(const Smem& sm, int team_size, int e) {
    int lo = 0, hi = team_size;  // invariant: prefix[lo] <= e < prefix[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (sm.prefix[mid] <= e) lo = mid; else hi = mid;
    }
    return lo;
}

// Second half of an insert in arrival-order mode: the claiming thread takes the next local id and publishes it.
template <typename PtrT>
__device__ __forceinline__ int arrival_assign(const KParams& p, const Hop& h, const Table& tab, int g, int r) {
    cg::coalesced_group grp = cg::coalesced_threads();  // one atomicAdd per group of claiming lanes
    int base = 0;
    if (grp.thread_rank() == 0) base = atomicAdd(h.counts + h.hop + 1, (int)grp.size());
    base = grp.shfl(base, 0);
    const int local = base + (int)grp.thread_rank();
    const uint32_t pos = (uint32_t)~r;
    if ((int64_t)local < h.nodes_cap) {
        h.nodes[local] = g;
        if (h.node_deg && !h.last_hop && (int64_t)local < h.deg_cap) {
            long long start;
            int deg;
            load_adj<PtrT>(p, g, start, deg);
            __stcg(h.node_start + local, start);
            __stcg(h.node_deg + local, deg);
        }
        atomicExch(tab.slots + pos, ((unsigned long long)(uint32_t)g << 32) | (uint32_t)local);
        return local;
    }
    set_status(p.status, FGL_ERR_CAPACITY);
    atomicExch(tab.slots + pos, ((unsigned long long)(uint32_t)g << 32));
    return 0;
}

// One sampled edge of the wide-fanout path: picked source `g` of seed `v`, edge number e within the hop.
// first_cnt counts the edges of this thread that may be first occurrences (fused, first-occurrence order).
template <typename PtrT, int MODE, bool ARRIVAL>
__device__ __forceinline__ void emit_edge(const KParams& p, const Hop& h, const Table& tab, const Smem& sm, int team_size,
                                          int32_t* team_cnt, int v, int g, int e, int& first_cnt) {
    if (MODE == MODE_SAMPLE) {
        h.blk_src[e] = g;
        if (h.out_dst) h.out_dst[e] = v;
        return;
    }
    if (g < 0 || (int64_t)g >= p.n_nodes) {
        set_status(p.status, FGL_ERR_BOUNDS);
        h.blk_src[e] = 0;
        return;
    }
    if (ARRIVAL) {
        bool created;
        int r = table_insert<true>(tab, (uint32_t)g, (uint32_t)e, p.status, created);
        if (created) r = arrival_assign<PtrT>(p, h, tab, g, r);
        h.blk_src[e] = r;
    } else {
        bool created;
        int displaced;
        int r = table_insert_track(tab, (uint32_t)g, (uint32_t)e, hash_pos(tab, (uint32_t)g), p.status, created, displaced);
        if (r < 0 && (created || displaced >= 0)) {
            r = ~((~r) | kTentative);
            ++first_cnt;
            if (displaced >= 0) atomicAdd(team_cnt + edge_owner(sm, team_size, displaced), -1);
        }
        h.blk_src[e] = r;
    }
}

// Fanouts up to 32: a group of G lanes per seed, one lane per pick; a group works on kSeedsPerIter seeds at a time.
// Stage 0, picks: every lane draws its own Philox word; for a k-subset (Floyd's algorithm: slot i draws t in
// [0, deg-k+i] and takes deg-k+i instead if an earlier slot already holds t) the group walks the slots in order, lane i
// settling slot i after a ballot over the earlier lanes -- the picks never leave the registers.  Stages 1-4 issue the
// dependent loads of the group's seeds stage by stage -- picked sources, first table probes, claims -- so that
// kSeedsPerIter independent round trips are in flight per lane instead of one chain after the other.
#ifndef FGL_SM_KS
#define FGL_SM_KS 4
#endif
constexpr int kSeedsPerIter = FGL_SM_KS;
constexpr int kGroupPathMaxFanout = 32;

template <typename PtrT, int MODE, bool ARRIVAL, int G>
__device__ __forceinline__ void sample_tile_groups(const KParams& p, const Hop& h, const Table& tab, Smem& sm, int team_size,
                                                   int32_t* team_cnt, int tile0, int tile_n, int& first_cnt) {
    const bool replace = (p.flags & FGL_SAMPLE_REPLACE) != 0;
    const int fanout = h.fanout;
    constexpr int kGroups = kThreads / G;
    constexpr int KS = kSeedsPerIter;
    const int gid = threadIdx.x / G, gl = threadIdx.x % G;
    const int gbase = (threadIdx.x & 31) & ~(G - 1);  // first lane of the group within its warp
    const unsigned gmask = G == 32 ? 0xffffffffu : ((1u << G) - 1u);
    for (int it = 0; it * kGroups * KS < tile_n; ++it) {
        int v[KS], off[KS], g[KS], deg[KS];
        long long start[KS];
        bool has[KS], hub[KS];
        uint32_t pk[KS], draw[KS];
        // stage 0: the picks
        bool any_hub = false;
#pragma unroll
        for (int q = 0; q < KS; ++q) {
            const int j = (it * KS + q) * kGroups + gid;
            v[q] = 0;
            off[q] = 0;
            g[q] = 0;
            deg[q] = 0;
            start[q] = 0;
            if (j < tile_n) {
                deg[q] = sm.deg[j];
                v[q] = sm.v[j];
                off[q] = sm.off[j];
                start[q] = sm.start[j];
            }
            has[q] = gl < min(deg[q], fanout);
            hub[q] = deg[q] > fanout;
            pk[q] = (uint32_t)gl;
            draw[q] = 0;
            if (hub[q] && gl < fanout) {
                draw[q] = philox_draw(p.rng_seed, h.ctr, (uint32_t)(tile0 + (it * KS + q) * kGroups + gid), (uint32_t)gl);
                if (replace) pk[q] = __umulhi(draw[q], (uint32_t)deg[q]);
            }
            any_hub |= hub[q];
        }
        if (!replace && __any_sync(0xffffffffu, any_hub)) {  // warp-uniform
            for (int i = 0; i < fanout; ++i) {
#pragma unroll
                for (int q = 0; q < KS; ++q) {
                    const uint32_t ri = __shfl_sync(0xffffffffu, draw[q], gbase + i);
                    const uint32_t jj = (uint32_t)(deg[q] - fanout + i);
                    const uint32_t tt = __umulhi(ri, jj + 1u);
                    const unsigned same = __ballot_sync(0xffffffffu, hub[q] && gl < i && pk[q] == tt);
                    if (hub[q] && gl == i) pk[q] = ((same >> gbase) & gmask) ? jj : tt;
                }
            }
        }
        // stage 1: the picked sources
#pragma unroll
        for (int q = 0; q < KS; ++q)
            if (has[q]) g[q] = ld_adjacency(p.indices + start[q] + (long long)pk[q]);
        if (MODE == MODE_SAMPLE) {
#pragma unroll
            for (int q = 0; q < KS; ++q) {
                if (has[q]) {
                    h.blk_src[off[q] + gl] = g[q];
                    if (h.out_dst) h.out_dst[off[q] + gl] = v[q];
                }
            }
        } else {
        // stage 2: first probe of every source
        uint32_t pos[KS];
        unsigned long long cur[KS], seen[KS];
#pragma unroll
        for (int q = 0; q < KS; ++q) {
            if (has[q] && (g[q] < 0 || (int64_t)g[q] >= p.n_nodes)) {
                set_status(p.status, FGL_ERR_BOUNDS);
                h.blk_src[off[q] + gl] = 0;
                has[q] = false;
            }
            pos[q] = hash_pos(tab, (uint32_t)g[q]);
            cur[q] = has[q] ? ld_slot(tab.slots + pos[q]) : 0ULL;
        }
        // stage 3: claim the slots that looked empty
#pragma unroll
        for (int q = 0; q < KS; ++q) {
            seen[q] = cur[q];
            if (has[q] && cur[q] == kEmpty) {
                const uint32_t e = (uint32_t)(off[q] + gl);
                seen[q] = atomicCAS(tab.slots + pos[q], kEmpty,
                                    ((unsigned long long)(uint32_t)g[q] << 32) | (ARRIVAL ? kPending : (kPending | e)));
            }
        }
        // stage 4: settle every edge; collisions continue probing one by one
#pragma unroll
        for (int q = 0; q < KS; ++q) {
            if (!has[q]) continue;
            const uint32_t key = (uint32_t)g[q];
            const int e = off[q] + gl;
            bool created = false;
            int displaced = -1;
            int r;
            if (cur[q] == kEmpty && seen[q] == kEmpty) {
                created = true;
                r = ~(int)pos[q];
            } else if ((uint32_t)(seen[q] >> 32) == key) {
                const uint32_t lo = (uint32_t)seen[q];
                if (!(lo & kPending)) {
                    r = (int)lo;
                } else {
                    if (!ARRIVAL && lo > (kPending | (uint32_t)e)) displaced = table_lower_edge(tab, pos[q], key, (uint32_t)e);
                    r = ~(int)pos[q];
                }
            } else if (ARRIVAL) {
                r = table_insert_from<true>(tab, key, (uint32_t)e, (pos[q] + 1) & tab.mask, p.status, created);
            } else {
                r = table_insert_track(tab, key, (uint32_t)e, (pos[q] + 1) & tab.mask, p.status, created, displaced);
            }
            if (ARRIVAL) {
                if (created) r = arrival_assign<PtrT>(p, h, tab, g[q], r);
            } else if (r < 0 && (created || displaced >= 0)) {
                r = ~((~r) | kTentative);
                ++first_cnt;
                if (displaced >= 0) atomicAdd(team_cnt + edge_owner(sm, team_size, displaced), -1);
            }
            h.blk_src[e] = r;
        }
        }  // MODE != MODE_SAMPLE
    }
}

// Any fanout up to FGL_MAX_FANOUT: one warp per seed, picks in shared memory.
template <typename PtrT, int MODE, bool ARRIVAL>
__device__ __forceinline__ void sample_tile_wide(const KParams& p, const Hop& h, const Table& tab, Smem& sm, int team_size,
                                                 int32_t* team_cnt, uint32_t* picks_all, int tile0, int tile_n, int& first_cnt) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool replace = (p.flags & FGL_SAMPLE_REPLACE) != 0;
    const int fanout = h.fanout;
    uint32_t* picks = picks_all + (size_t)warp * fanout;
    for (int j = warp; j < tile_n; j += kWarps) {
        const int v = sm.v[j], deg = sm.deg[j], off = sm.off[j];
        const long long start = sm.start[j];
        if (deg <= fanout) {
            for (int i = lane; i < deg; i += 32)
                emit_edge<PtrT, MODE, ARRIVAL>(p, h, tab, sm, team_size, team_cnt, v, p.indices[start + i], off + i, first_cnt);
        } else if (replace) {
            for (int i = lane; i < fanout; i += 32) {
                const uint32_t r = philox_draw(p.rng_seed, h.ctr, (uint32_t)(tile0 + j), (uint32_t)i);
                emit_edge<PtrT, MODE, ARRIVAL>(p, h, tab, sm, team_size, team_cnt, v,
                                               ld_adjacency(p.indices + start + (long long)__umulhi(r, (uint32_t)deg)), off + i, first_cnt);
            }
        } else {
            uint32_t r = 0;
            for (int i = 0; i < fanout; ++i) {
                if ((i & 31) == 0) {
                    r = (i + lane < fanout) ? philox_draw(p.rng_seed, h.ctr, (uint32_t)(tile0 + j), (uint32_t)(i + lane)) : 0u;
                }
                const uint32_t ri = __shfl_sync(0xffffffffu, r, i & 31);
                const uint32_t jj = (uint32_t)(deg - fanout + i);
                const uint32_t t = __umulhi(ri, jj + 1u);
                bool hit = false;
                for (int q = lane; q < i; q += 32) hit |= (picks[q] == t);
                const bool any = __any_sync(0xffffffffu, hit);
                if (lane == 0) picks[i] = any ? jj : t;
                __syncwarp();
            }
            for (int i = lane; i < fanout; i += 32)
                emit_edge<PtrT, MODE, ARRIVAL>(p, h, tab, sm, team_size, team_cnt, v, ld_adjacency(p.indices + start + (long long)picks[i]), off + i,
                                               first_cnt);
        }
        __syncwarp();
    }
}

// Phase A of the drop-in sampler: per-CTA sum of min(deg, fanout) over the CTA's slice of the seeds.
template <typename PtrT>
__device__ __forceinline__ void phase_count_seeds(const KParams& p, const Hop& h, const Team& t, Smem& sm,
                                                  int32_t* team_sums) {
    int s0, s1;
    chunk_of(h.n_seeds, t.rank, t.size, s0, s1);
    int acc = 0;
    for (int s = s0 + (int)threadIdx.x; s < s1; s += 4 * kThreads) {
        int v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] = (s + q * kThreads < s1) ? __ldcg(h.nodes + s + q * kThreads) : -1;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (s + q * kThreads < s1) {
                long long start;
                int deg;
                load_adj<PtrT>(p, v[q], start, deg);
                acc += min(deg, h.fanout);
            }
        }
    }
    const int total = block_sum(acc, sm.scan);
    if (threadIdx.x == 0) __stcg(team_sums + t.rank, total);
}

// Phase A of the fused kernel: the same sum from the degrees cached when the nodes joined the list (coalesced);
// also resets this CTA's count of first occurrences.
__device__ __forceinline__ void phase_count_cached(const Hop& h, const Team& t, Smem& sm, int32_t* team_sums, int32_t* team_cnt) {
    int s0, s1;
    chunk_of(h.n_seeds, t.rank, t.size, s0, s1);
    int acc = 0;
    for (int s = s0 + (int)threadIdx.x; s < s1; s += kThreads) acc += min(__ldcg(h.node_deg + s), h.fanout);
    const int total = block_sum(acc, sm.scan);
    if (threadIdx.x == 0) {
        __stcg(team_sums + t.rank, total);
        __stcg(team_cnt + t.rank, 0);
    }
}

// Sum of the team's partials before `rank` and over the whole team.
__device__ __forceinline__ void team_prefix(const int32_t* team_sums, const Team& t, Smem& sm, int& before, int& total) {
    int a = 0, b = 0;
    for (int q = threadIdx.x; q < t.size; q += kThreads) {
        const int x = __ldcg(team_sums + q);
        b += x;
        if (q < t.rank) a += x;
    }
    before = block_sum(a, sm.scan);
    total = block_sum(b, sm.scan);
}

// Phase B: offsets, picks, source reads, table inserts.  Returns the CTA's first edge and edge count.
template <typename PtrT, int MODE, bool ARRIVAL>
__device__ __forceinline__ void phase_sample(const KParams& p, const Hop& h, const Table& tab, const Team& t,
                                             Smem& sm, uint32_t* picks, const int32_t* team_sums, int32_t* team_cnt, int& e0,
                                             int& e1, int& e_total) {
    int before, total;
    if (MODE == MODE_FUSED) {
        // the edge ranges of all CTAs of the team (an edge number's owner is looked up when it is displaced)
        const int x = (int)threadIdx.x < t.size ? __ldcg(team_sums + threadIdx.x) : 0;
        const int excl = block_excl_scan(x, sm.scan, total);
        if ((int)threadIdx.x < t.size) sm.prefix[threadIdx.x] = excl;
        if (threadIdx.x == 0) sm.prefix[t.size] = total;
        __syncthreads();
        before = sm.prefix[t.rank];
    } else {
        team_prefix(team_sums, t, sm, before, total);
    }
    e_total = total;
    int s0, s1;
    chunk_of(h.n_seeds, t.rank, t.size, s0, s1);
    if (t.rank == 0 && threadIdx.x == 0) {
        h.counts[8 + h.hop] = total;
        if (h.blk_indptr) h.blk_indptr[h.n_seeds] = total;
    }
    int running = before;
    int first_cnt = 0;
    e0 = before;
    for (int tile0 = s0; tile0 < s1; tile0 += kThreads) {
        const int s = tile0 + (int)threadIdx.x;
        int k = 0;
        if (s < s1) {
            const int v = __ldcg(h.nodes + s);
            long long start;
            int deg;
            if (MODE == MODE_FUSED) {
                start = __ldcg(h.node_start + s);
                deg = __ldcg(h.node_deg + s);
            } else {
                load_adj<PtrT>(p, v, start, deg);
            }
            k = min(deg, h.fanout);
            sm.v[threadIdx.x] = v;
            sm.start[threadIdx.x] = start;
            sm.deg[threadIdx.x] = deg;
        }
        int tile_total;
        const int excl = block_excl_scan(k, sm.scan, tile_total);
        if (s < s1) {
            sm.off[threadIdx.x] = running + excl;
            if (h.blk_indptr) h.blk_indptr[s] = running + excl;
        }
        __syncthreads();
        const int tile_n = min(kThreads, s1 - tile0);
        if (h.fanout <= 8)
            sample_tile_groups<PtrT, MODE, ARRIVAL, 8>(p, h, tab, sm, t.size, team_cnt, tile0, tile_n, first_cnt);
        else if (h.fanout <= 16)
            sample_tile_groups<PtrT, MODE, ARRIVAL, 16>(p, h, tab, sm, t.size, team_cnt, tile0, tile_n, first_cnt);
        else if (h.fanout <= kGroupPathMaxFanout)
            sample_tile_groups<PtrT, MODE, ARRIVAL, 32>(p, h, tab, sm, t.size, team_cnt, tile0, tile_n, first_cnt);
        else
            sample_tile_wide<PtrT, MODE, ARRIVAL>(p, h, tab, sm, t.size, team_cnt, picks, tile0, tile_n, first_cnt);
        running += tile_total;
        __syncthreads();
    }
    e1 = running;
    if (MODE == MODE_FUSED && !ARRIVAL) {
        const int mine = block_sum(first_cnt, sm.scan);
        if (threadIdx.x == 0 && mine != 0) atomicAdd(team_cnt + t.rank, mine);
    }
}

// ---- fused kernel, first-occurrence order ------------------------------------------------------------------------------
// Phase D: the possibly-first edges that still hold their slot are the first occurrences.  Local ids in edge order;
// the node, its adjacency offset and degree (unless this is the last hop) join the list; the edge entry becomes the id.
// Eight consecutive edges per thread: two 128-bit loads of entries, then up to eight slot loads in flight.
template <typename PtrT>
__device__ __forceinline__ int phase_rank_tracked(const KParams& p, const Hop& h, const Table& tab, int32_t* edges, int e0, int e1,
                                                  int n_before, const Team& t, Smem& sm, const int32_t* team_cnt) {
    int before, total;
    team_prefix(team_cnt, t, sm, before, total);
    int running = n_before + before;
    constexpr int kPer = 8;
    for (int tile0 = e0 & ~3; tile0 < e1; tile0 += kPer * kThreads) {
        const int eb = tile0 + kPer * (int)threadIdx.x;
        int m[kPer];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int at = eb + 4 * half;
            int4 x = make_int4(0, 0, 0, 0);
            if (at + 3 >= e0 && at + 3 < e1) {
                x = __ldcg(reinterpret_cast<const int4*>(edges + at));  // the row is 16-byte aligned
            } else if (at < e1 && at + 3 >= e0) {  // the range's last entries: never read beyond e1
                x.x = __ldcg(edges + at);
                if (at + 1 < e1) x.y = __ldcg(edges + at + 1);
                if (at + 2 < e1) x.z = __ldcg(edges + at + 2);
            }
            m[4 * half + 0] = x.x;
            m[4 * half + 1] = x.y;
            m[4 * half + 2] = x.z;
            m[4 * half + 3] = x.w;
        }
        unsigned long long cur[kPer];
#pragma unroll
        for (int q = 0; q < kPer; ++q) {
            const bool mine = eb + q >= e0 && eb + q < e1 && m[q] < 0 && ((~m[q]) & kTentative);
            if (!mine) m[q] = 0;
            cur[q] = mine ? ld_slot(tab.slots + ((~m[q]) & kSlotMask)) : 0ULL;
        }
        int firsts = 0;
#pragma unroll
        for (int q = 0; q < kPer; ++q) {
            if (!(m[q] < 0 && (uint32_t)cur[q] == (kPending | (uint32_t)(eb + q)))) m[q] = 0;  // keep first occurrences
            firsts += m[q] < 0 ? 1 : 0;
        }
        int tile_total;
        int local = running + block_excl_scan(firsts, sm.scan, tile_total);
#pragma unroll
        for (int q = 0; q < kPer; ++q) {
            if (m[q] < 0) {
                const uint32_t pos = (uint32_t)((~m[q]) & kSlotMask);
                const uint32_t key = (uint32_t)(cur[q] >> 32);
                if ((int64_t)local < h.nodes_cap) {
                    h.nodes[local] = (int)key;
                    tab.slots[pos] = ((unsigned long long)key << 32) | (uint32_t)local;
                    edges[eb + q] = local;
                    if (!h.last_hop && (int64_t)local < h.deg_cap) {
                        long long start;
                        int deg;
                        load_adj<PtrT>(p, (int)key, start, deg);
                        __stcg(h.node_start + local, start);
                        __stcg(h.node_deg + local, deg);
                    }
                } else {
                    set_status(p.status, FGL_ERR_CAPACITY);
                    tab.slots[pos] = ((unsigned long long)key << 32);
                    edges[eb + q] = 0;
                }
                ++local;
            }
        }
        running += tile_total;
    }
    return n_before + total;
}

// Phase E: the entries that are still pending take the local id their slot now holds.
__device__ __forceinline__ void phase_relabel_tracked(const Table& tab, int32_t* edges, int e0, int e1) {
    constexpr int kPer = 8;
    for (int tile0 = e0 & ~3; tile0 < e1; tile0 += kPer * kThreads) {
        const int eb = tile0 + kPer * (int)threadIdx.x;
        int m[kPer];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int at = eb + 4 * half;
            int4 x = make_int4(0, 0, 0, 0);
            if (at + 3 >= e0 && at + 3 < e1) {
                x = __ldcg(reinterpret_cast<const int4*>(edges + at));
            } else if (at < e1 && at + 3 >= e0) {  // the range's last entries: never read beyond e1
                x.x = __ldcg(edges + at);
                if (at + 1 < e1) x.y = __ldcg(edges + at + 1);
                if (at + 2 < e1) x.z = __ldcg(edges + at + 2);
            }
            m[4 * half + 0] = x.x;
            m[4 * half + 1] = x.y;
            m[4 * half + 2] = x.z;
            m[4 * half + 3] = x.w;
        }
        unsigned long long cur[kPer];
#pragma unroll
        for (int q = 0; q < kPer; ++q) {
            const bool mine = eb + q >= e0 && eb + q < e1 && m[q] < 0;
            if (!mine) m[q] = 0;
            cur[q] = mine ? ld_slot(tab.slots + ((~m[q]) & kSlotMask)) : 0ULL;
        }
#pragma unroll
        for (int q = 0; q < kPer; ++q)
            if (m[q] < 0) edges[eb + q] = (int)((uint32_t)cur[q] & ~kPending);
    }
}

// ---- drop-in id map (fgl_map): counting pass, rank, relabel over entries that are local ids or ~slot --------------------
// Phase C: number of first occurrences among the CTA's edges.
__device__ __forceinline__ void phase_count_first(const Table& tab, const int32_t* edges, int e0, int e1, const Team& t,
                                                  Smem& sm, int32_t* team_sums) {
    int acc = 0;
    for (int e = e0 + (int)threadIdx.x; e < e1; e += 4 * kThreads) {
        int m[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) m[q] = (e + q * kThreads < e1) ? __ldcg(edges + e + q * kThreads) : 0;
        unsigned long long cur[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) cur[q] = (m[q] < 0) ? ld_slot(tab.slots + (uint32_t)~m[q]) : 0ULL;
#pragma unroll
        for (int q = 0; q < 4; ++q)
            acc += (m[q] < 0 && (uint32_t)cur[q] == (kPending | (uint32_t)(e + q * kThreads))) ? 1 : 0;
    }
    const int total = block_sum(acc, sm.scan);
    if (threadIdx.x == 0) __stcg(team_sums + t.rank, total);
}

// Phase D: local ids in first-occurrence order; returns the new node count.
__device__ __forceinline__ int phase_rank(const KParams& p, const Table& tab, const int32_t* edges, int e0, int e1,
                                          int32_t* nodes, int64_t nodes_cap, int n_before, const Team& t, Smem& sm,
                                          const int32_t* team_sums) {
    int before, total;
    team_prefix(team_sums, t, sm, before, total);
    int running = n_before + before;
    // every thread ranks four consecutive edges: their entries and slots are loaded together
    for (int tile0 = e0; tile0 < e1; tile0 += 4 * kThreads) {
        const int eb = tile0 + 4 * (int)threadIdx.x;
        int m[4];
        unsigned long long cur[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) m[q] = (eb + q < e1) ? __ldcg(edges + eb + q) : 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) cur[q] = (m[q] < 0) ? ld_slot(tab.slots + (uint32_t)~m[q]) : 0ULL;
        int mine = 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (!(m[q] < 0 && (uint32_t)cur[q] == (kPending | (uint32_t)(eb + q)))) m[q] = 0;  // keep first occurrences
            mine += m[q] < 0 ? 1 : 0;
        }
        int tile_total;
        int local = running + block_excl_scan(mine, sm.scan, tile_total);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (m[q] < 0) {
                const uint32_t pos = (uint32_t)~m[q];
                const uint32_t key = (uint32_t)(cur[q] >> 32);
                if ((int64_t)local < nodes_cap) {
                    nodes[local] = (int)key;
                    tab.slots[pos] = ((unsigned long long)key << 32) | (uint32_t)local;
                } else {
                    set_status(p.status, FGL_ERR_CAPACITY);
                    tab.slots[pos] = ((unsigned long long)key << 32);
                }
                ++local;
            }
        }
        running += tile_total;
    }
    return n_before + total;
}

// Phase E: slot positions -> local ids.
__device__ __forceinline__ void phase_relabel(const Table& tab, int32_t* edges, int e0, int e1) {
    for (int e = e0 + (int)threadIdx.x; e < e1; e += 4 * kThreads) {
        int m[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) m[q] = (e + q * kThreads < e1) ? __ldcg(edges + e + q * kThreads) : 0;
        unsigned long long cur[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) cur[q] = (m[q] < 0) ? ld_slot(tab.slots + (uint32_t)~m[q]) : 0ULL;
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (m[q] < 0) edges[e + q * kThreads] = (int)((uint32_t)cur[q] & ~kPending);
    }
}

// ----------------------------------------------------------------------------------------------
// kernels
// ----------------------------------------------------------------------------------------------
template <typename PtrT, int MODE, bool ARRIVAL>
__global__ void __launch_bounds__(kThreads, kMinCtas) sample_map_kernel(const __grid_constant__ KParams p) {
    __shared__ Smem sm;
    extern __shared__ uint32_t picks[];
    const int team_id = blockIdx.x / p.team_size;
    if (team_id >= p.n_teams) return;
    if (*(volatile int32_t*)(p.status + 1) != 0) return;  // an earlier launch gave up: wait for fgl_ws_check
    Team t;
    t.rank = blockIdx.x % p.team_size;
    t.size = p.team_size;
    t.epoch = 0;
    t.bar = p.barriers + (size_t)team_id * 16;
    t.status = p.status;
    int32_t* team_sums = p.team_sums + (size_t)team_id * p.team_size;
    int32_t* team_cnt = p.team_cnt + (size_t)team_id * p.team_size;
    Table tab;
    tab.slots = p.table + (size_t)team_id * (size_t)p.table_slots;
    tab.mask = (uint32_t)(p.table_slots - 1);
    tab.shift = p.table_shift;

    for (int b = team_id; b < p.n_batches; b += p.n_teams) {
        Hop h;
        h.nodes = p.nodes + (size_t)b * p.nodes_stride;
        h.nodes_cap = p.nodes_stride;
        h.counts = p.counts + (size_t)b * FGL_COUNTS_STRIDE;
        h.out_dst = p.out_dst;
        h.node_start = nullptr;
        h.node_deg = nullptr;
        h.deg_cap = 0;
        int n0 = p.seed_counts ? __ldg(p.seed_counts + b) : p.n_seeds_host;
        n0 = max(0, min(n0, (int)min((int64_t)0x7fffffff, p.seed_stride)));
        const int32_t* seeds = p.seeds + (size_t)b * p.seed_stride;

        if (MODE == MODE_FUSED) {
            // The team's table is empty here: the host cleared it once and every mini-batch clears it again at its
            // end.  Insert the seeds with local id = position; cache their adjacency offsets and degrees.
            h.node_start = p.node_start + (size_t)team_id * p.deg_stride;
            h.node_deg = p.node_deg + (size_t)team_id * p.deg_stride;
            h.deg_cap = p.deg_stride;
            if (t.rank == 0 && threadIdx.x < FGL_COUNTS_STRIDE) h.counts[threadIdx.x] = threadIdx.x == 0 ? n0 : 0;
            int s0, s1;
            chunk_of(n0, t.rank, t.size, s0, s1);
            for (int s = s0 + (int)threadIdx.x; s < s1; s += kThreads) {
                const int v = seeds[s];
                h.nodes[s] = v;
                long long start = 0;
                int deg = 0;
                if (v < 0 || (int64_t)v >= p.n_nodes) {
                    set_status(p.status, FGL_ERR_BOUNDS);
                } else {
                    table_insert_seed(tab, (uint32_t)v, (uint32_t)s, p.status);
                    load_adj<PtrT>(p, v, start, deg);
                }
                __stcg(h.node_start + s, start);
                __stcg(h.node_deg + s, deg);
            }
            // the same CTA (the same thread, even) reads these entries back in phases A and B of the first hop, so no
            // barrier is needed before them; the barrier after phase A orders the seed inserts before the first
            // source insert
        } else {
            h.nodes = const_cast<int32_t*>(seeds);  // MODE_SAMPLE reads the seeds in place
        }

        int n_cur = n0;
        for (int hop = 0; hop < p.n_hops; ++hop) {
            h.hop = hop;
            h.last_hop = hop + 1 == p.n_hops;
            h.fanout = p.fanout[hop];
            h.n_seeds = n_cur;
            h.ctr = p.rng_ctr + (uint64_t)b * 8u + (uint64_t)hop;
            h.blk_indptr = p.blk_indptr[hop] ? p.blk_indptr[hop] + (size_t)b * p.blk_indptr_stride[hop] : nullptr;
            h.blk_src = p.blk_src[hop] + (size_t)b * p.blk_src_stride[hop];

            if (MODE == MODE_FUSED)
                phase_count_cached(h, t, sm, team_sums, team_cnt);
            else
                phase_count_seeds<PtrT>(p, h, t, sm, team_sums);
            if (MODE == MODE_FUSED && ARRIVAL && t.rank == 0 && threadIdx.x == 0) h.counts[hop + 1] = n_cur;
            if (!team_barrier(t, &sm.flag)) return;

            int e0, e1, e_total;
            phase_sample<PtrT, MODE, ARRIVAL>(p, h, tab, t, sm, picks, team_sums, team_cnt, e0, e1, e_total);
            if (MODE == MODE_SAMPLE) break;
            if (!team_barrier(t, &sm.flag)) return;

            if (!ARRIVAL) {
                n_cur = phase_rank_tracked<PtrT>(p, h, tab, h.blk_src, e0, e1, n_cur, t, sm, team_cnt);
                n_cur = (int)min((int64_t)n_cur, h.nodes_cap);
                if (t.rank == 0 && threadIdx.x == 0) h.counts[hop + 1] = n_cur;
                if (!team_barrier(t, &sm.flag)) return;
                phase_relabel_tracked(tab, h.blk_src, e0, e1);
            } else {
                n_cur = (int)min((int64_t)__ldcg(h.counts + hop + 1), h.nodes_cap);
                phase_relabel(tab, h.blk_src, e0, e1);
            }
            // the next hop's phase A only reads the degrees cached before the last barrier; its barrier keeps the
            // next inserts behind every CTA's relabel reads
        }
        if (MODE == MODE_SAMPLE) break;
        // Once every CTA has finished reading the table, clear it for the next mini-batch: a coalesced sweep of the
        // team's (L2-resident) slots.
        if (!team_barrier(t, &sm.flag)) return;
        {
            const int64_t vecs = p.table_slots / 2;  // two slots per 128-bit store
            uint4* base = reinterpret_cast<uint4*>(tab.slots);
            const uint4 ones = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
            for (int64_t i = (int64_t)t.rank * kThreads + threadIdx.x; i < vecs; i += (int64_t)t.size * kThreads) base[i] = ones;
        }
        if (b + p.n_teams < p.n_batches) {
            if (!team_barrier(t, &sm.flag)) return;
        }
    }
}

// Explicit-edge mapping (the drop-in transfer_edge_id).  The table was cleared by the host.
template <bool ARRIVAL>
__global__ void __launch_bounds__(kThreads, kMinCtas) map_kernel(const __grid_constant__ KParams p) {
    __shared__ Smem sm;
    Team t;
    t.rank = blockIdx.x;
    t.size = gridDim.x;
    t.epoch = 0;
    t.bar = p.barriers;
    t.status = p.status;
    int32_t* team_sums = p.team_sums;
    Table tab;
    tab.slots = p.table;
    tab.mask = (uint32_t)(p.table_slots - 1);
    tab.shift = p.table_shift;
    const int n_seeds = p.n_seeds_host;
    const int n_edges = (int)p.map_edges;
    int32_t* unique = p.nodes;
    const int64_t nodes_cap = p.nodes_stride;

    int s0, s1;
    chunk_of(n_seeds, t.rank, t.size, s0, s1);
    for (int s = s0 + (int)threadIdx.x; s < s1; s += kThreads) {
        const int v = p.seeds[s];
        unique[s] = v;  // id_map.cu:285
        if (v < 0)
            set_status(p.status, FGL_ERR_BOUNDS);
        else
            table_insert_seed(tab, (uint32_t)v, (uint32_t)s, p.status);
    }
    if (t.rank == 0 && threadIdx.x == 0) p.counts[1] = n_seeds;
    if (!team_barrier(t, &sm.flag)) return;

    int e0, e1;
    chunk_of(n_edges, t.rank, t.size, e0, e1);
    for (int e = e0 + (int)threadIdx.x; e < e1; e += kThreads) {
        const int g = p.map_src[e];
        if (g < 0) {
            set_status(p.status, FGL_ERR_BOUNDS);
            p.map_src[e] = 0;
        } else {
            // same table as the fused kernel; n_nodes is not known here
            bool created;
            int r = table_insert<ARRIVAL>(tab, (uint32_t)g, (uint32_t)e, p.status, created);
            if (ARRIVAL && created) {
                cg::coalesced_group grp = cg::coalesced_threads();
                int base = 0;
                if (grp.thread_rank() == 0) base = atomicAdd(p.counts + 1, (int)grp.size());
                base = grp.shfl(base, 0);
                const int local = base + (int)grp.thread_rank();
                const uint32_t pos = (uint32_t)~r;
                if ((int64_t)local < nodes_cap) {
                    unique[local] = g;
                    atomicExch(tab.slots + pos, ((unsigned long long)(uint32_t)g << 32) | (uint32_t)local);
                    r = local;
                } else {
                    set_status(p.status, FGL_ERR_CAPACITY);
                    atomicExch(tab.slots + pos, ((unsigned long long)(uint32_t)g << 32));
                    r = 0;
                }
            }
            p.map_src[e] = r;
        }
        if (p.map_dst) {  // id_map.cu:378-381; the seeds all have their ids since the barrier
            const int d = p.map_dst[e];
            p.map_dst[e] = d < 0 ? 0 : table_lookup(tab, (uint32_t)d, p.status);
            if (d < 0) set_status(p.status, FGL_ERR_BOUNDS);
        }
    }
    if (!team_barrier(t, &sm.flag)) return;
    if (!ARRIVAL) {
        phase_count_first(tab, p.map_src, e0, e1, t, sm, team_sums);
        if (!team_barrier(t, &sm.flag)) return;
        const int n_total = phase_rank(p, tab, p.map_src, e0, e1, unique, nodes_cap, n_seeds, t, sm, team_sums);
        if (t.rank == 0 && threadIdx.x == 0) p.counts[1] = (int)min((int64_t)n_total, nodes_cap);
        if (!team_barrier(t, &sm.flag)) return;
    }
    phase_relabel(tab, p.map_src, e0, e1);
}

// ----------------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------------
static int64_t pow2_at_least(int64_t n) {
    int64_t p = 1024;
    while (p < n) p <<= 1;
    return p;
}

static int log2_of(int64_t pow2) {
    int l = 0;
    while ((1LL << l) < pow2) ++l;
    return l;
}

template <typename K>
static int max_coresident(Workspace* ws, K kernel, size_t dyn_smem, int* out) {
    if (dyn_smem > 48 * 1024)
        FGL_CUDA_OK(ws, cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn_smem));
    int per_sm = 0;
    FGL_CUDA_OK(ws, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, dyn_smem));
    if (per_sm < 1) {
        ws->last_error = "kernel does not fit on an SM";
        return FGL_ERR_CUDA;
    }
    *out = per_sm * ws->sm_count;
    return FGL_OK;
}

template <typename K>
static int launch_coop(Workspace* ws, K kernel, int grid, size_t dyn_smem, KParams* kp, cudaStream_t st) {
    if (dyn_smem > 48 * 1024)
        FGL_CUDA_OK(ws, cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn_smem));
    void* args[] = {(void*)kp};
    timing_begin(ws, st);
    const cudaError_t e = cudaLaunchCooperativeKernel((const void*)kernel, dim3(grid), dim3(kThreads), args, dyn_smem, st);
    timing_end(ws, st);
    FGL_CUDA_OK(ws, e);
    return FGL_OK;
}

// scratch layout: [barriers: n_teams * 16 u64][team_sums: grid i32][team_cnt: grid i32][counts: 16 i32]
//                 [node_start: n_teams * deg_stride i64][node_deg: n_teams * deg_stride i32]
// Only the part before node_start is zeroed per call.
static int64_t sums_bytes(int grid) { return (((int64_t)grid * 4 + 127) / 128) * 128; }

static int64_t scratch_head(int n_teams, int grid) { return (int64_t)n_teams * 128 + 2 * sums_bytes(grid) + 128; }

static int64_t scratch_need(int n_teams, int grid, int64_t deg_stride = 0) {
    return scratch_head(n_teams, grid) + (int64_t)n_teams * deg_stride * 12;
}

static void place_scratch(Workspace* ws, KParams& kp, int n_teams, int grid, int64_t deg_stride, int32_t** call_counts) {
    char* base = ws->scratch;
    kp.barriers = (unsigned long long*)base;
    kp.team_sums = (int32_t*)(base + (size_t)n_teams * 128);
    kp.team_cnt = (int32_t*)(base + (size_t)n_teams * 128 + sums_bytes(grid));
    if (call_counts) *call_counts = (int32_t*)(base + scratch_head(n_teams, grid) - 128);
    kp.node_start = (long long*)(base + scratch_head(n_teams, grid));
    kp.node_deg = (int32_t*)(base + scratch_head(n_teams, grid) + (size_t)n_teams * deg_stride * 8);
    kp.deg_stride = deg_stride;
    kp.status = ws->status;
}

template <int MODE>
static int launch_sample_map(Workspace* ws, KParams& kp, bool is64, bool arrival, int grid, size_t dyn, cudaStream_t st) {
#define FGL_LAUNCH(PT, AR) launch_coop(ws, sample_map_kernel<PT, MODE, AR>, grid, dyn, &kp, st)
    if (is64) return arrival ? FGL_LAUNCH(int64_t, true) : FGL_LAUNCH(int64_t, false);
    return arrival ? FGL_LAUNCH(int32_t, true) : FGL_LAUNCH(int32_t, false);
#undef FGL_LAUNCH
}

template <int MODE>
static int occupancy_sample_map(Workspace* ws, bool is64, bool arrival, size_t dyn, int* out) {
#define FGL_OCC(PT, AR) max_coresident(ws, sample_map_kernel<PT, MODE, AR>, dyn, out)
    if (is64) return arrival ? FGL_OCC(int64_t, true) : FGL_OCC(int64_t, false);
    return arrival ? FGL_OCC(int32_t, true) : FGL_OCC(int32_t, false);
#undef FGL_OCC
}

// dynamic shared memory: a row of picks per warp for fanouts beyond 32 (narrower fanouts keep their picks in registers)
static size_t picks_smem(int max_fanout) {
    return max_fanout > kGroupPathMaxFanout ? (size_t)kWarps * max_fanout * sizeof(uint32_t) : 0;
}

}  // namespace fgl

using namespace fgl;

extern "C" {

int fgl_fused_capacity(int64_t n_nodes, int32_t max_seeds, int32_t n_hops, const int32_t* fanout, int64_t* cap_nodes) {
    if (n_nodes <= 0 || max_seeds < 0 || n_hops < 1 || n_hops > FGL_MAX_HOPS || !fanout || !cap_nodes) return FGL_ERR_INVALID;
    cap_nodes[0] = max_seeds;
    for (int h = 0; h < n_hops; ++h) {
        if (fanout[h] < 1 || fanout[h] > FGL_MAX_FANOUT) return FGL_ERR_INVALID;
        const int64_t grown = cap_nodes[h] * (1 + (int64_t)fanout[h]);
        cap_nodes[h + 1] = std::max<int64_t>(cap_nodes[h], std::min<int64_t>(n_nodes, grown));
        if (cap_nodes[h] * (int64_t)fanout[h] > 0x7fffffffLL) return FGL_ERR_INVALID;
    }
    return FGL_OK;
}

int fgl_sample(fgl_ws* ws, const void* indptr, int indptr_is_64, const int32_t* indices, int64_t n_nodes,
               const int32_t* seeds, int32_t n_seeds, int32_t fanout, int32_t flags, uint64_t rng_seed,
               uint64_t rng_ctr, int32_t* out_indptr, int32_t* out_src, int32_t* out_dst, int64_t* n_edges_host,
               void* stream) {
    if (!ws || !indptr || !indices || n_nodes <= 0 || n_seeds < 0 || fanout < 1 || fanout > FGL_MAX_FANOUT ||
        (n_seeds > 0 && (!seeds || !out_src)) || (int64_t)n_seeds * fanout > 0x7fffffffLL)
        return FGL_ERR_INVALID;
    std::lock_guard<std::mutex> lock(ws->mu);
    DeviceGuard guard(ws->device);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t dyn = picks_smem(fanout);
    int max_grid = 0;
    int rc = occupancy_sample_map<MODE_SAMPLE>(ws, indptr_is_64 != 0, false, dyn, &max_grid);
    if (rc != FGL_OK) return rc;
    const int lanes = fanout <= 8 ? 8 : (fanout <= 16 ? 16 : 32);
    const int64_t seeds_per_cta = kThreads / lanes;
    int grid = (int)std::max<int64_t>(1, std::min<int64_t>(max_grid, (n_seeds + seeds_per_cta - 1) / seeds_per_cta));
    rc = ws_ensure(ws, 0, scratch_need(1, grid));
    if (rc != FGL_OK) return rc;
    KParams kp;
    std::memset(&kp, 0, sizeof(kp));
    int32_t* call_counts = nullptr;
    place_scratch(ws, kp, 1, grid, 0, &call_counts);
    kp.indptr = indptr;
    kp.indices = indices;
    kp.n_nodes = n_nodes;
    kp.n_batches = 1;
    kp.n_hops = 1;
    kp.fanout[0] = fanout;
    kp.flags = flags;
    kp.n_teams = 1;
    kp.team_size = grid;
    kp.rng_seed = rng_seed;
    kp.rng_ctr = rng_ctr;
    kp.seeds = seeds;
    kp.seed_stride = n_seeds;
    kp.seed_counts = nullptr;
    kp.n_seeds_host = n_seeds;
    kp.nodes = nullptr;
    kp.nodes_stride = n_seeds;
    kp.counts = call_counts;
    kp.blk_indptr[0] = out_indptr;
    kp.blk_src[0] = out_src;
    kp.out_dst = out_dst;
    kp.table = nullptr;
    kp.table_slots = 1024;
    kp.table_shift = 22;
    FGL_CUDA_OK(ws, cudaMemsetAsync(ws->scratch, 0, (size_t)scratch_head(1, grid), st));
    rc = launch_sample_map<MODE_SAMPLE>(ws, kp, indptr_is_64 != 0, false, grid, dyn, st);
    if (rc != FGL_OK) return rc;
    if (n_edges_host) {
        FGL_CUDA_OK(ws, cudaMemcpyAsync(ws->host_pinned, call_counts + 8, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
        FGL_CUDA_OK(ws, cudaMemcpyAsync(ws->host_pinned + 1, ws->status, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
        FGL_CUDA_OK(ws, cudaStreamSynchronize(st));
        *n_edges_host = ws->host_pinned[0];
        const int code = ws->host_pinned[1];
        if (code != FGL_OK) {
            FGL_CUDA_OK(ws, cudaMemsetAsync(ws->status, 0, 2 * sizeof(int32_t), st));
            ws->last_error = std::string("fgl_sample: ") + fgl_status_str(code);
            return code;
        }
    }
    return FGL_OK;
}

int fgl_map(fgl_ws* ws, int32_t* src, int32_t* dst, const int32_t* seeds, int32_t n_seeds, int64_t n_edges,
            int32_t* unique, int64_t unique_cap, int32_t flags, int64_t* n_unique_host, void* stream) {
    if (!ws || n_seeds < 0 || n_edges < 0 || n_edges > 0x7fffffffLL || (n_seeds > 0 && !seeds) || (n_edges > 0 && !src) ||
        !unique || unique_cap < n_seeds)
        return FGL_ERR_INVALID;
    std::lock_guard<std::mutex> lock(ws->mu);
    DeviceGuard guard(ws->device);
    cudaStream_t st = (cudaStream_t)stream;
    const bool arrival = (flags & FGL_MAP_ARRIVAL_ORDER) != 0;
    int max_grid = 0;
    int rc = arrival ? max_coresident(ws, map_kernel<true>, 0, &max_grid) : max_coresident(ws, map_kernel<false>, 0, &max_grid);
    if (rc != FGL_OK) return rc;
    const int64_t work = std::max<int64_t>(n_edges, n_seeds);
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(max_grid, (work + 2 * kThreads - 1) / (2 * kThreads)));
    // at most n_seeds + min(n_edges, unique_cap - n_seeds) distinct keys; load factor <= 2/3
    const int64_t max_keys = (int64_t)n_seeds + n_edges;
    const int64_t slots = pow2_at_least(max_keys + max_keys / 2 + 1);
    if (slots > (1LL << 31)) return FGL_ERR_CAPACITY;
    rc = ws_ensure(ws, slots, scratch_need(1, grid));
    if (rc != FGL_OK) return rc;
    KParams kp;
    std::memset(&kp, 0, sizeof(kp));
    int32_t* call_counts = nullptr;
    place_scratch(ws, kp, 1, grid, 0, &call_counts);
    kp.n_nodes = 0x7fffffff;
    kp.flags = flags;
    kp.n_teams = 1;
    kp.team_size = grid;
    kp.seeds = seeds;
    kp.n_seeds_host = n_seeds;
    kp.nodes = unique;
    kp.nodes_stride = unique_cap;
    kp.counts = call_counts;
    kp.map_src = src;
    kp.map_dst = dst;
    kp.map_edges = n_edges;
    kp.table = ws->table;
    kp.table_slots = slots;
    kp.table_shift = 32 - log2_of(slots);
    FGL_CUDA_OK(ws, cudaMemsetAsync(ws->scratch, 0, (size_t)scratch_head(1, grid), st));
    FGL_CUDA_OK(ws, cudaMemsetAsync(ws->table, 0xFF, sizeof(unsigned long long) * (size_t)slots, st));
    ws->table_dirty = true;  // this call leaves its keys in the table
    rc = arrival ? launch_coop(ws, map_kernel<true>, grid, 0, &kp, st) : launch_coop(ws, map_kernel<false>, grid, 0, &kp, st);
    if (rc != FGL_OK) return rc;
    if (n_unique_host) {
        FGL_CUDA_OK(ws, cudaMemcpyAsync(ws->host_pinned, call_counts + 1, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
        FGL_CUDA_OK(ws, cudaMemcpyAsync(ws->host_pinned + 1, ws->status, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
        FGL_CUDA_OK(ws, cudaStreamSynchronize(st));
        *n_unique_host = ws->host_pinned[0];
        const int code = ws->host_pinned[1];
        if (code != FGL_OK) {
            FGL_CUDA_OK(ws, cudaMemsetAsync(ws->status, 0, 2 * sizeof(int32_t), st));
            ws->last_error = std::string("fgl_map: ") + fgl_status_str(code);
            return code;
        }
    }
    return FGL_OK;
}

int fgl_sample_map_fused(fgl_ws* ws, const fgl_fused_args* a, void* stream) {
    if (!ws || !a || !a->indptr || !a->indices || a->n_nodes <= 0 || a->n_batches < 0 || a->n_hops < 1 ||
        a->n_hops > FGL_MAX_HOPS || !a->seeds || !a->seed_counts || !a->nodes || !a->counts || a->seed_stride < 0)
        return FGL_ERR_INVALID;
    if (a->n_batches == 0) return FGL_OK;
    int64_t cap[FGL_MAX_HOPS + 1];
    if (a->seed_stride > 0x7fffffffLL) return FGL_ERR_INVALID;
    int rc = fgl_fused_capacity(a->n_nodes, (int32_t)a->seed_stride, a->n_hops, a->fanout, cap);
    if (rc != FGL_OK) return rc;
    int max_fanout = 0;
    for (int h = 0; h < a->n_hops; ++h) {
        max_fanout = std::max(max_fanout, (int)a->fanout[h]);
        if (!a->block_indptr[h] || !a->block_src[h] || a->block_indptr_stride[h] < cap[h] + 1 ||
            a->block_src_stride[h] < cap[h] * a->fanout[h])
            return FGL_ERR_INVALID;
    }
    if (a->nodes_stride < cap[a->n_hops]) return FGL_ERR_INVALID;
    for (int h = 0; h < a->n_hops; ++h)   // the relabelling passes read and write the edge entries four at a time
        if (((uintptr_t)a->block_src[h] & 15) != 0 || a->block_src_stride[h] % 4 != 0) return FGL_ERR_INVALID;
    const int64_t deg_stride = (cap[a->n_hops - 1] + 31) / 32 * 32;   // nodes that can still become seeds
    std::lock_guard<std::mutex> lock(ws->mu);
    DeviceGuard guard(ws->device);
    cudaStream_t st = (cudaStream_t)stream;
    const bool arrival = (a->flags & FGL_MAP_ARRIVAL_ORDER) != 0;
    const bool is64 = a->indptr_is_64 != 0;
    const size_t dyn = picks_smem(max_fanout);
    int max_grid = 0;
    rc = occupancy_sample_map<MODE_FUSED>(ws, is64, arrival, dyn, &max_grid);
    if (rc != FGL_OK) return rc;
    int n_teams = a->n_teams > 0 ? a->n_teams : 4;
    n_teams = std::max(1, std::min(std::min(n_teams, (int)a->n_batches), max_grid));
    const int team_size = max_grid / n_teams;
    const int grid = team_size * n_teams;
    // one table per team: sized for the worst case, or by the caller's hint (a smaller table stays in L2;
    // if it fills up the launch reports FGL_ERR_PROBE and the caller retries without a hint)
    int64_t slots = pow2_at_least(cap[a->n_hops] + cap[a->n_hops] / 2 + 1);
    if (a->table_slots_hint > 0) slots = std::min(slots, pow2_at_least(a->table_slots_hint));
    if (slots > (1LL << 29)) return FGL_ERR_CAPACITY;   // pending edge entries keep a slot number in 29 bits
    if (team_size > kMaxTeam) return FGL_ERR_INVALID;
    rc = ws_ensure(ws, slots * n_teams, scratch_need(n_teams, grid, deg_stride));
    if (rc != FGL_OK) return rc;
    if (ws->table_dirty) {
        FGL_CUDA_OK(ws, cudaMemsetAsync(ws->table, 0xFF, sizeof(unsigned long long) * (size_t)ws->table_slots, st));
        ws->table_dirty = false;
    }
    KParams kp;
    std::memset(&kp, 0, sizeof(kp));
    place_scratch(ws, kp, n_teams, grid, deg_stride, nullptr);
    kp.indptr = a->indptr;
    kp.indices = a->indices;
    kp.n_nodes = a->n_nodes;
    kp.n_batches = a->n_batches;
    kp.n_hops = a->n_hops;
    for (int h = 0; h < a->n_hops; ++h) {
        kp.fanout[h] = a->fanout[h];
        kp.blk_indptr[h] = a->block_indptr[h];
        kp.blk_indptr_stride[h] = a->block_indptr_stride[h];
        kp.blk_src[h] = a->block_src[h];
        kp.blk_src_stride[h] = a->block_src_stride[h];
    }
    kp.flags = a->flags;
    kp.n_teams = n_teams;
    kp.team_size = team_size;
    kp.rng_seed = a->rng_seed;
    kp.rng_ctr = a->rng_ctr;
    kp.seeds = a->seeds;
    kp.seed_stride = a->seed_stride;
    kp.seed_counts = a->seed_counts;
    kp.nodes = a->nodes;
    kp.nodes_stride = a->nodes_stride;
    kp.counts = a->counts;
    kp.table = ws->table;
    kp.table_slots = slots;
    kp.table_shift = 32 - log2_of(slots);
    FGL_CUDA_OK(ws, cudaMemsetAsync(ws->scratch, 0, (size_t)scratch_head(n_teams, grid), st));
    return launch_sample_map<MODE_FUSED>(ws, kp, is64, arrival, grid, dyn, st);
}

}  // extern "C"
