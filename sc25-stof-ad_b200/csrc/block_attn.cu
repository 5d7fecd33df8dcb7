// Block-masked multi-head attention for sm_100a: TMA-fed tcgen05 MMAs with the accumulators in tensor
// memory, online softmax in registers, only listed K/V blocks ever loaded.
//
// Tiling.  A work item is a PAIR of 64-row halves of one (batch, head) - two 64-row stretches of the sequence, neighbours
// by default.  Each half walks its own list of 64-wide K/V tiles (the tiles any of its row blocks lists): all products are
// M = 64 tcgen05 MMAs, whose 64 accumulator rows occupy lanes 0-15 of each 32-lane quarter of tensor memory; half A's
// products are placed there and half B's 16 lanes further up, so that together they fill the 128 lanes and every softmax
// warp (one quarter: 16 rows of A, 16 rows of B) has work at every step, whatever the two lists have in common.  Step j of
// an item works on tile A[j] for half A and tile B[j] for half B; tiles both halves list come first, at the same step, and
// are loaded once, and such a step runs as ONE M = 128 product on a copy of Q whose rows are interleaved the way the lanes are
// (full tensor-core rate; M = 64 products take the time of M = 128 ones).  Block sizes 16..128 are mapped onto this tiling by a PLAN built once per block index (plan_kernel): per
// item the two tile lists step by step and, per step, one code for each 16-row x 16-column group (0 absent, 1 full, 2+i
// partial tile i of the row block).
//
// Kernel.  Persistent, two thread blocks per SM, static schedule over the items (heavy items first inside groups of
// (batch, head) pairs small enough to keep their K/V in L2, dealt round-robin; or a table made by the caller that balances the
// step counts over the thread blocks).
//   warp 4      TMA producer: Q of the next item (its two 64-row halves, and the same rows interleaved), K tiles through a ring of four slots, V
//               tiles through a ring of three (one slot per step when both halves use the same tile, else two)
//   warp 5      MMA issuer:   S = Q K^T (64 x 64 x 64 per half) into one of THREE S buffers in tensor memory, up to three steps
//               ahead of the PV products; O += P V per half with P read back from tensor memory (fp16) and V consumed in its
//               natural key-row-major layout through an MN-major descriptor
//   warps 0-3   softmax: one query row per thread (tensor-memory lane): tcgen05.ld of the scores, masking from the plan
//               codes, row maximum (3-input max), exp2 with scale and maximum folded into packed FMAs (part of the
//               exponentials on the FMA pipe by polynomial), lazy rescale of O (only when the maximum grew by more than
//               2^8), P written with tcgen05.st, final O / l normalisation staged in shared memory and written with TMA stores
// With three S buffers the QK^T products run ahead of the softmax warps.  Masking of partial tiles and the rescale of O are
// out-of-line functions that work on tensor memory in place.  Tiles nobody lists are never loaded.
#include <atomic>
#include "stof_host.h"
#include "stof_ptx.cuh"

namespace stof {
namespace {

constexpr int A_TQ = 128, A_TKV = 64, A_D = 64;
constexpr int A_HALF = 64;                        // rows of one half (one M = 64 product)
#ifndef A_SBUF_N
#define A_SBUF_N 3
#endif
#ifndef A_KSLOTS_N
#define A_KSLOTS_N 4
#endif
#ifndef A_VSLOTS_N
#define A_VSLOTS_N 3
#endif
#ifndef A_QBUFS_N
#define A_QBUFS_N 1
#endif
constexpr int A_SBUF = A_SBUF_N;                  // S buffers in tensor memory: QK^T runs up to this many steps ahead of PV
constexpr int A_KSLOTS = A_KSLOTS_N, A_VSLOTS = A_VSLOTS_N;   // K and V rings (a step takes one slot of each, or two)
constexpr int A_QBUFS = A_QBUFS_N;                // Q buffers (items in flight on the QK^T side)
// "tile(s) of step s have landed" barriers are counted per STEP (one wait per step for the MMA issuer, whether the step brought
// one tile or two), "slot free" barriers per ring slot.  A full barrier is armed again A_FBARS steps later; by then its ring
// slots have been handed back, which the issuer does only after it has seen the barrier complete: A_FBARS >= ring slots.
constexpr int A_FBARS = A_KSLOTS > A_VSLOTS ? A_KSLOTS : A_VSLOTS;
constexpr int A_Q_BYTES = A_TQ * A_D * 2;         // 16 KB: the two halves of an item, 8 KB each
// A Q buffer holds the item's rows twice: half A then half B (the operands of the per-half M = 64 products), and the same rows
// interleaved in chunks of 16 - A0-15, B0-15, A16-31, ... - which as the operand of ONE M = 128 product puts every row into the
// tensor-memory lane the per-half products put it in; steps in which both halves work on the same key tile use that form.
constexpr int A_QBUF_BYTES = 2 * A_Q_BYTES;
constexpr int A_KV_BYTES = A_TKV * A_D * 2;       // 8 KB per K or V tile
constexpr int A_OSTAGE_BYTES = 32 * A_D * 2;     // 4 KB output staging per softmax warp (TMA store source)
constexpr int A_THREADS = 192;
constexpr int A_CTAS_PER_SM = 2;
constexpr int A_TMEM_COLS = 256;
constexpr int A_COL_S = 0, A_COL_O = A_SBUF * A_TKV;         // S0 @0, S1 @64, S2 @128 (P overlays the first 32 columns of its S), O @192
constexpr uint32_t A_LANE_B = 16u << 16;          // tensor-memory address offset of half B's lanes inside each quarter
constexpr int A_MAX_TABLE_BYTES = 48 * 1024;
constexpr float A_RESCALE_THRESHOLD = 8.0f;       // log2 units
#ifndef A_POLY_PAIRS
#define A_POLY_PAIRS 2                            // of every 8 column pairs, this many take the polynomial exp2
#endif
constexpr int A_GROUP_BH = 40;                    // (batch, head) pairs per scheduling group: 40 x 2 x S x 128 B of K/V stay in L2
constexpr unsigned A_NO_TILE = 0xFFFFu;           // "this half has no tile at this step"

enum {
    AB_Q_FULL = 0, AB_Q_EMPTY = A_QBUFS, AB_O_FREE = 2 * A_QBUFS, AB_S_FULL = AB_O_FREE + 1, AB_P_FULL = AB_S_FULL + A_SBUF, AB_PV_DONE = AB_P_FULL + A_SBUF,
    AB_K_FULL = AB_PV_DONE + A_SBUF, AB_K_EMPTY = AB_K_FULL + A_FBARS, AB_V_FULL = AB_K_EMPTY + A_KSLOTS,
    AB_V_EMPTY = AB_V_FULL + A_FBARS, AB_COUNT = AB_V_EMPTY + A_VSLOTS
};

// ---------------------------------------------------------------------------------------------
// Plan layout (all offsets from the start of the plan buffer, 16-byte aligned sections)
// ---------------------------------------------------------------------------------------------
struct PlanHeader {
    int magic, seq_len, bm, bn;
    int n_qtiles, max_steps, total_steps, reserved;
};
constexpr int PLAN_MAGIC = 0x53544F47;
__host__ __device__ inline size_t plan_off_nsteps() { return sizeof(PlanHeader); }
__host__ __device__ inline size_t plan_off_order(int nqt) { return plan_off_nsteps() + ((static_cast<size_t>(nqt) * 4 + 15) & ~static_cast<size_t>(15)); }
// per (item, step): tile of half A in the low 16 bits, tile of half B in the high 16 bits (A_NO_TILE: none)
__host__ __device__ inline size_t plan_off_steps(int nqt) { return plan_off_order(nqt) + ((static_cast<size_t>(nqt) * 8 + 15) & ~static_cast<size_t>(15)); }
__host__ __device__ inline size_t plan_off_codes(int nqt, int maxs) {
    return plan_off_steps(nqt) + ((static_cast<size_t>(nqt) * maxs * 4 + 15) & ~static_cast<size_t>(15));
}
// first sequence row of the two 64-row halves of each item (int2; y = -1 when the item has one half only)
__host__ __device__ inline size_t plan_off_halves(int nqt, int maxs) { return plan_off_codes(nqt, maxs) + static_cast<size_t>(nqt) * maxs * 64; }
__host__ __device__ inline size_t plan_total_bytes(int nqt, int maxs) {
    return plan_off_halves(nqt, maxs) + ((static_cast<size_t>(nqt) * 8 + 15) & ~static_cast<size_t>(15));
}

// One thread block per item: code table in shared memory -> the two halves' tile lists, aligned step by step, + 8x4 group
// codes per step.  An item is two 64-row halves of the sequence: halves 2t and 2t + 1 by default, or the two that `pairs`
// names for it (a caller pairs halves with equally long lists, so that neither waits for the other).
// The last block to finish ranks the items by step count (descending, stable) for the scheduler.
__global__ void __launch_bounds__(256)
plan_kernel(const int* __restrict__ full_row_ptr, const int* __restrict__ full_col_idx, const int* __restrict__ part_row_ptr,
            const int* __restrict__ part_col_idx, const int2* __restrict__ pairs, int seq_len, int bm, int bn, unsigned char* plan,
            unsigned int* ticket, int* status) {
    extern __shared__ uint16_t table[];                 // [2 halves x row blocks per half][ncb], then three tile lists of maxt entries
    __shared__ int s_ns, s_na, s_nb;
    __shared__ bool s_last;
    const int nqt = gridDim.x, maxt = (seq_len + A_TKV - 1) / A_TKV;
    const int qt = blockIdx.x;
    const int nbm = seq_len / bm, ncb = seq_len / bn;
    const int nrbh = bm >= 64 ? 1 : 64 / bm, nrb = 2 * nrbh;        // table rows per half, per item
    uint16_t* list_s = table + nrb * ncb;                           // tiles both halves list (ascending)
    uint16_t* list_a = list_s + maxt;                               // tiles only half A lists
    uint16_t* list_b = list_a + maxt;                               // tiles only half B lists
    const int n_half = (seq_len + 63) / 64;
    int half[2] = {2 * qt, 2 * qt + 1 < n_half ? 2 * qt + 1 : -1};
    if (pairs != nullptr) {
        const int2 pr = pairs[qt];
        if (pr.x >= 0 && pr.x < n_half && pr.y >= -1 && pr.y < n_half && pr.x != pr.y) {
            half[0] = pr.x; half[1] = pr.y;
        } else {
            if (status && threadIdx.x == 0) atomicCAS(status, 0, STATUS_BAD_INDEX);
            half[0] = 0; half[1] = -1;
        }
    }
    int* n_steps = reinterpret_cast<int*>(plan + plan_off_nsteps());
    int2* order = reinterpret_cast<int2*>(plan + plan_off_order(nqt));     // per rank: {item, step count}
    uint32_t* steps = reinterpret_cast<uint32_t*>(plan + plan_off_steps(nqt)) + static_cast<size_t>(qt) * maxt;
    uint16_t* codes = reinterpret_cast<uint16_t*>(plan + plan_off_codes(nqt, maxt)) + static_cast<size_t>(qt) * maxt * 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    for (int i = threadIdx.x; i < nrb * ncb; i += blockDim.x) table[i] = 0;
    __syncthreads();
    for (int lrb = 0; lrb < nrb; ++lrb) {
        const int hb = half[lrb / nrbh];
        if (hb < 0) continue;
        const int rb = bm >= 64 ? (hb * 64) / bm : hb * nrbh + lrb % nrbh;
        if (rb >= nbm) continue;
        const int f0 = full_row_ptr[rb], f1 = full_row_ptr[rb + 1];
        for (int i = f0 + threadIdx.x; i < f1; i += blockDim.x) {
            const int c = full_col_idx[i];
            if (c >= 0 && c < ncb) table[lrb * ncb + c] = 1;
            else if (status) atomicCAS(status, 0, STATUS_BAD_INDEX);
        }
        const int p0 = part_row_ptr[rb], p1 = part_row_ptr[rb + 1];
        for (int i = p0 + threadIdx.x; i < p1; i += blockDim.x) {
            const int c = part_col_idx[i];
            if (c >= 0 && c < ncb && i - p0 < 16382) table[lrb * ncb + c] = static_cast<uint16_t>(2 + (i - p0));     // 14-bit codes
            else if (status) atomicCAS(status, 0, STATUS_BAD_INDEX);
        }
    }
    __syncthreads();
    if (warp == 0) {
        int ns = 0, na = 0, nb = 0;
        for (int t0 = 0; t0 < maxt; t0 += 32) {
            const int t = t0 + lane;
            bool act[2] = {false, false};
            if (t < maxt) {
                const int c_lo = (t * A_TKV) / bn;
                const int c_hi = min(ncb - 1, (t * A_TKV + A_TKV - 1) / bn);
                for (int lrb = 0; lrb < nrb; ++lrb)
                    for (int c = c_lo; c <= c_hi; ++c) act[lrb / nrbh] |= table[lrb * ncb + c] != 0;
            }
            const unsigned lower = (1u << lane) - 1u;
            const unsigned bal_s = __ballot_sync(0xffffffffu, act[0] && act[1]);
            const unsigned bal_a = __ballot_sync(0xffffffffu, act[0] && !act[1]);
            const unsigned bal_b = __ballot_sync(0xffffffffu, !act[0] && act[1]);
            if (act[0] && act[1]) list_s[ns + __popc(bal_s & lower)] = static_cast<uint16_t>(t);
            if (act[0] && !act[1]) list_a[na + __popc(bal_a & lower)] = static_cast<uint16_t>(t);
            if (!act[0] && act[1]) list_b[nb + __popc(bal_b & lower)] = static_cast<uint16_t>(t);
            ns += __popc(bal_s);
            na += __popc(bal_a);
            nb += __popc(bal_b);
        }
        if (lane == 0) {
            s_ns = ns; s_na = na; s_nb = nb;
            n_steps[qt] = ns + max(na, nb);
        }
    }
    __syncthreads();
    const int ns = s_ns, na = s_na, nb = s_nb;
    const int count = ns + max(na, nb);
    // tile of half h at step j: the tiles both halves list come first, then each half's own
    auto step_tile = [&](int j, int h) -> unsigned {
        if (j < ns) return list_s[j];
        const int i = j - ns;
        if (h == 0) return i < na ? list_a[i] : A_NO_TILE;
        return i < nb ? list_b[i] : A_NO_TILE;
    };
    for (int j = threadIdx.x; j < count; j += blockDim.x) steps[j] = step_tile(j, 0) | (step_tile(j, 1) << 16);
    // codes[j][row group 0..7][col group 0..3], 14 bits each; row group = 4 * half + quarter, i.e. the 16 rows of that half
    // that live in softmax warp `quarter`.  The top two bits of the LAST code of a row group carry the class of that warp at
    // this step (its two row groups x four column groups): 0 every group absent, 1 every row group either full or - its half
    // having no tile at this step - absent, 2 anything else: the kernel then needs no warp vote to pick its path.
    auto group_row = [&](int rg) { return half[rg >> 2] < 0 ? -1 : half[rg >> 2] * 64 + (rg & 3) * 16; };
    auto table_row = [&](int rg) { return (rg >> 2) * nrbh + (bm >= 64 ? 0 : ((rg & 3) * 16) / bm); };
    auto group_code = [&](int j, int rg, int cg) -> uint16_t {
        const unsigned t = step_tile(j, rg >> 2);
        if (t == A_NO_TILE) return 0;
        const int row = group_row(rg), col = static_cast<int>(t) * A_TKV + cg * 16;
        return (row >= 0 && row < seq_len && col < seq_len) ? table[table_row(rg) * ncb + col / bn] : uint16_t(0);
    };
    for (int i = threadIdx.x; i < count * 32; i += blockDim.x) {
        const int j = i >> 5, rg = (i >> 2) & 7, cg = i & 3;
        uint16_t code = group_code(j, rg, cg);
        if (cg == 3) {
            bool all0 = true, fast = true;
            for (int r2 = (rg & 3); r2 < 8; r2 += 4) {
                bool g0 = true, g1 = true;
                for (int c2 = 0; c2 < 4; ++c2) {
                    const uint16_t k2 = group_code(j, r2, c2);
                    g0 &= k2 == 0;
                    g1 &= k2 == 1;
                }
                all0 &= g0;
                fast &= g1 || (g0 && step_tile(j, r2 >> 2) == A_NO_TILE);
            }
            code = static_cast<uint16_t>(code | ((all0 ? 0u : (fast ? 1u : 2u)) << 14));
        }
        codes[i] = code;
    }
    if (threadIdx.x == 0)
        reinterpret_cast<int2*>(plan + plan_off_halves(nqt, maxt))[qt] = make_int2(half[0] * 64, half[1] < 0 ? -1 : half[1] * 64);
    // the last block orders the items by descending step count (stable)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(ticket, 1u);
        s_last = (t == gridDim.x - 1);
        if (s_last) *ticket = 0;
    }
    __syncthreads();
    if (s_last) {
        __threadfence();
        PlanHeader* h = reinterpret_cast<PlanHeader*>(plan);
        int total = 0;
        for (int a = threadIdx.x; a < nqt; a += blockDim.x) {
            const int na2 = __ldcg(n_steps + a);
            int rank = 0;
            for (int b = 0; b < nqt; ++b) {
                const int nb2 = __ldcg(n_steps + b);
                rank += (nb2 > na2 || (nb2 == na2 && b < a)) ? 1 : 0;
            }
            order[rank] = make_int2(a, na2);
            total += na2;
        }
        atomicAdd(&h->total_steps, total);
        if (threadIdx.x == 0) {
            h->magic = PLAN_MAGIC; h->seq_len = seq_len; h->bm = bm; h->bn = bn;
            h->n_qtiles = nqt; h->max_steps = maxt; h->reserved = 0;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Attention kernel
// ---------------------------------------------------------------------------------------------
struct AttnParams {
    const int* part_row_ptr;
    const __half* part_block_mask;
    const unsigned char* plan;
    int batch, heads, seq_len;
    int bm, bn, bm_shift, bn_shift;
    int n_qtiles, max_steps;
    unsigned total_items, bh_total;
    int slot_s[4], slot_h[4], slot_b[4];   // coordinate slot (1..3) of row / head / batch in the q, k, v, out tensor maps
    float scale_log2;
    int* status;
    const int* schedule;                   // optional caller-made deal of the items to the thread blocks (see fetch_item)
};

__device__ __forceinline__ void tma_tile(void* dst, const CUtensorMap* map, uint64_t* bar, int row, int h, int b, int ss, int sh, int sb) {
    const int c1 = ss == 1 ? row : (sh == 1 ? h : b);
    const int c2 = ss == 2 ? row : (sh == 2 ? h : b);
    const int c3 = ss == 3 ? row : (sh == 3 ? h : b);
    tma_load_4d(dst, map, bar, 0, c1, c2, c3);
}

__device__ __forceinline__ void tma_tile_store(const CUtensorMap* map, const void* src, int row, int h, int b, int ss, int sh, int sb) {
    const int c1 = ss == 1 ? row : (sh == 1 ? h : b);
    const int c2 = ss == 2 ? row : (sh == 2 ? h : b);
    const int c3 = ss == 3 ? row : (sh == 3 ? h : b);
    tma_store_4d(map, src, 0, c1, c2, c3);
}

// Static schedule.  Default: items are enumerated group by group ((batch, head) pairs in chunks of A_GROUP_BH), inside a
// group in rank order (the items with the most steps first), and dealt round-robin to the thread blocks.  With a schedule table
// ({blocks G, G + 1 offsets, item ids = (batch * heads + head) * query tiles + query tile}, made by the caller, e.g. by a
// longest-processing-time assignment over the tile counts) block b walks ids[offset[b] .. offset[b + 1]).
struct Item {
    int qt, head, batch, n;
    bool valid;
};
// Where this thread block's items come from: its stretch of the schedule table (read once), or the round-robin deal.
struct ItemSource {
    const int* ids;          // the block's item numbers in the caller's table (nullptr: default deal)
    unsigned count;          // how many items the block has
};
__device__ __forceinline__ ItemSource item_source(const AttnParams& p) {
    ItemSource src;
    if (p.schedule != nullptr) {
        const int b0 = __ldg(p.schedule + 1 + blockIdx.x), b1 = __ldg(p.schedule + 2 + blockIdx.x);
        src.ids = p.schedule + 2 + gridDim.x + b0;
        src.count = b1 > b0 ? static_cast<unsigned>(b1 - b0) : 0u;
    } else {
        src.ids = nullptr;
        src.count = blockIdx.x < p.total_items ? (p.total_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
    }
    return src;
}
// Step one of fetching item k of this thread block: its raw number (A_NO_ITEM when the block has no k-th item).
constexpr unsigned A_NO_ITEM = 0xffffffffu;
__device__ __forceinline__ unsigned fetch_item_id(unsigned k, const ItemSource& src) {
    if (k >= src.count) return A_NO_ITEM;
    return src.ids != nullptr ? static_cast<unsigned>(__ldg(src.ids + k)) : blockIdx.x + k * gridDim.x;
}
// Step two: the item's coordinates and its tile count.
__device__ __forceinline__ Item decode_item(unsigned id, const AttnParams& p, const int2* sched) {
    Item it;
    it.qt = 0; it.head = 0; it.batch = 0; it.n = 0;
    it.valid = id != A_NO_ITEM;
    if (!it.valid) return it;
    if (p.schedule != nullptr) {
        if (id >= p.total_items) {                       // a table that does not belong to this launch: stop, and say so
            if (p.status) atomicCAS(p.status, 0, STATUS_BAD_INDEX);
            it.valid = false;
            return it;
        }
        const unsigned bh = id / static_cast<unsigned>(p.n_qtiles);
        it.qt = static_cast<int>(id - bh * static_cast<unsigned>(p.n_qtiles));
        it.n = __ldg(reinterpret_cast<const int*>(p.plan + plan_off_nsteps()) + it.qt);
        it.batch = static_cast<int>(bh / p.heads);
        it.head = static_cast<int>(bh - it.batch * p.heads);
        return it;
    }
    const unsigned group_items = static_cast<unsigned>(A_GROUP_BH) * p.n_qtiles;
    const unsigned g = id / group_items;
    const unsigned r = id - g * group_items;
    const unsigned bh0 = g * A_GROUP_BH;
    const unsigned gsize = min(static_cast<unsigned>(A_GROUP_BH), p.bh_total - bh0);     // the tail group is smaller
    const unsigned rank = r / gsize;
    const unsigned bh = bh0 + (r - rank * gsize);
    const int2 sc = __ldg(sched + rank);
    it.qt = sc.x;
    it.n = sc.y;
    it.batch = static_cast<int>(bh / p.heads);
    it.head = static_cast<int>(bh - it.batch * p.heads);
    return it;
}
__device__ __forceinline__ Item fetch_item(unsigned k, const ItemSource& src, const AttnParams& p, const int2* sched) {
    return decode_item(fetch_item_id(k, src), p, sched);
}
// The items of a thread block in order, fetched ahead of use: an item's number is requested two items early and decoded (which
// asks for its step count) one item early, so that moving on to the next item waits for no load.  Items without steps are
// skipped by the callers that only deal with steps (`skip_empty`).
struct ItemQueue {
    ItemSource src;
    unsigned k;              // index of `cur` among the block's items
    Item cur, nxt;
    unsigned id2;
    __device__ __forceinline__ void init(const AttnParams& p, const int2* sched) {
        src = item_source(p);
        k = 0;
        cur = fetch_item(0, src, p, sched);
        nxt = fetch_item(1, src, p, sched);
        id2 = fetch_item_id(2, src);
    }
    __device__ __forceinline__ void pop(const AttnParams& p, const int2* sched) {
        ++k;
        cur = nxt;
        nxt = decode_item(id2, p, sched);
        id2 = fetch_item_id(k + 2, src);
    }
    __device__ __forceinline__ void skip_empty(const AttnParams& p, const int2* sched) {
        while (cur.valid && cur.n == 0) pop(p, sched);
    }
};

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Rare paths of the softmax loop are kept out of line (and work on tensor memory, not on the caller's register arrays) so that
// the loop the warps spend their time in stays a few kilobytes of straight-line code.

// Address of the 16 mask addends (fp16) of this thread's row in column group cg of a partial block (code c >= 2)
__device__ __forceinline__ const __half* mask_row_ptr(const __half* part_block_mask, int part_base, unsigned c, int bm_shift, int bn,
                                                      int row_in_block, int col) {
    return part_block_mask + ((static_cast<size_t>(part_base + c - 2) << bm_shift) + row_in_block) * bn + (col & (bn - 1));
}

// Applies the block mask to the 32 x 64 scores of one warp in place: column groups a row does not list become -inf, partial
// groups get their -10000 * (1 - mask) addend.  `cx`, `cy` hold this thread's four group codes.
__device__ __noinline__ void mask_scores_in_tmem(uint32_t t_s, uint32_t cx, uint32_t cy, const __half* part_block_mask, int part_base, int bm_shift,
                                                 int bn, int row_in_block, int col0) {
    const unsigned code[4] = {cx & 0xFFFFu, cx >> 16, cy & 0xFFFFu, (cy >> 16) & 0x3FFFu};     // the top bits of the last code hold the warp class
    uint4 m[4][2];                                                 // all addends are requested before the first is used
#pragma unroll
    for (int cg = 0; cg < 4; ++cg) {
        m[cg][0] = make_uint4(0u, 0u, 0u, 0u);
        m[cg][1] = make_uint4(0u, 0u, 0u, 0u);
        if (code[cg] >= 2u) {
            const __half* mp = mask_row_ptr(part_block_mask, part_base, code[cg], bm_shift, bn, row_in_block, col0 + cg * 16);
            m[cg][0] = __ldg(reinterpret_cast<const uint4*>(mp));
            m[cg][1] = __ldg(reinterpret_cast<const uint4*>(mp + 8));
        }
    }
#pragma unroll
    for (int cg = 0; cg < 4; ++cg) {
        const unsigned c = code[cg];
        if (__all_sync(0xffffffffu, c == 1u)) continue;
        uint32_t v[16];
        tmem_ld16(t_s + cg * 16, v);
        tc_wait_ld();
        if (c == 0u) {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0xFF800000u;      // -inf
        } else if (c >= 2u) {
            const __half2* h0 = reinterpret_cast<const __half2*>(&m[cg][0]);
            const __half2* h1 = reinterpret_cast<const __half2*>(&m[cg][1]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 a = __half22float2(h0[i]), b = __half22float2(h1[i]);
                v[2 * i] = __float_as_uint(__uint_as_float(v[2 * i]) + a.x);
                v[2 * i + 1] = __float_as_uint(__uint_as_float(v[2 * i + 1]) + a.y);
                v[8 + 2 * i] = __float_as_uint(__uint_as_float(v[8 + 2 * i]) + b.x);
                v[8 + 2 * i + 1] = __float_as_uint(__uint_as_float(v[8 + 2 * i + 1]) + b.y);
            }
        }
        tmem_st16(t_s + cg * 16, v);
    }
    tc_wait_st();
}

// O *= alpha for this thread's row (64 fp32 columns in tensor memory)
__device__ __noinline__ void rescale_o_in_tmem(uint32_t t_o, float alpha) {
#pragma unroll 1
    for (int c = 0; c < A_D; c += 16) {
        uint32_t o[16];
        tmem_ld16(t_o + c, o);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st16(t_o + c, o);
    }
    tc_wait_st();
}

// The four K = 16 products of one 64 x 64 x 64 block, issued as one instruction sequence (the issuing thread is a single lane:
// every instruction it spends between two products delays all of them).
// S[tmem] = Q[smem] K[smem]^T: both K-major operands advance by 32 bytes (2 in descriptor units) per product.
__device__ __forceinline__ void mma_chain_qk(uint32_t d_tmem, uint64_t q_desc, uint64_t k_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p0, p1;\n\t.reg .b64 a, b;\n\t"
        "setp.ne.b32 p0, 0, 0;\n\t"
        "setp.eq.b32 p1, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n\t"
        "add.s64 a, %1, 2;\n\tadd.s64 b, %2, 2;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
        "add.s64 a, %1, 4;\n\tadd.s64 b, %2, 4;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
        "add.s64 a, %1, 6;\n\tadd.s64 b, %2, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t}"
        ::"r"(d_tmem), "l"(q_desc), "l"(k_desc), "r"(idesc)
        : "memory");
}
// O[tmem] (+)= P[tmem] V[smem]: P advances by 8 columns (16 fp16 keys) per product, the MN-major V by 16 key rows = 2048 bytes
// (128 in descriptor units); `accumulate` = 0 overwrites O with the first product.
__device__ __forceinline__ void mma_chain_pv(uint32_t o_tmem, uint32_t p_tmem, uint64_t v_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p0, p1;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
        "setp.ne.b32 p0, %4, 0;\n\t"
        "setp.eq.b32 p1, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
        "add.u32 a, %1, 8;\n\tadd.s64 b, %2, 128;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, p1;\n\t"
        "add.u32 a, %1, 16;\n\tadd.s64 b, %2, 256;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, p1;\n\t"
        "add.u32 a, %1, 24;\n\tadd.s64 b, %2, 384;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, p1;\n\t}"
        ::"r"(o_tmem), "r"(p_tmem), "l"(v_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(A_THREADS, A_CTAS_PER_SM)
block_attn_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_q16, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, const AttnParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* q_smem = smem;                                   // 2 buffers
    unsigned char* k_smem = q_smem + A_QBUFS * A_QBUF_BYTES;
    unsigned char* v_smem = k_smem + A_KSLOTS * A_KV_BYTES;
    unsigned char* o_smem = v_smem + A_VSLOTS * A_KV_BYTES;          // 4 x 4 KB, one slab per softmax warp
    uint64_t* bars = reinterpret_cast<uint64_t*>(o_smem + 4 * A_OSTAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + AB_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const WaitCtx wctx{abort_flag, p.status};
    const int2* plan_sched = reinterpret_cast<const int2*>(p.plan + plan_off_order(p.n_qtiles));
    const uint32_t* plan_steps = reinterpret_cast<const uint32_t*>(p.plan + plan_off_steps(p.n_qtiles));
    const uint16_t* plan_codes = reinterpret_cast<const uint16_t*>(p.plan + plan_off_codes(p.n_qtiles, p.max_steps));
    const int2* plan_halves = reinterpret_cast<const int2*>(p.plan + plan_off_halves(p.n_qtiles, p.max_steps));

    if (threadIdx.x == 0) {
        // a plan made for another sequence length or block shape is reported, not followed
        const int4 ph = __ldg(reinterpret_cast<const int4*>(p.plan));
        const int st = p.status != nullptr ? *p.status : 0;
        for (int i = 0; i < A_QBUFS; ++i) {
            mbar_init(&bars[AB_Q_FULL + i], 1);
            mbar_init(&bars[AB_Q_EMPTY + i], 1);
        }
        mbar_init(&bars[AB_O_FREE], 4);
        for (int i = 0; i < A_SBUF; ++i) {
            mbar_init(&bars[AB_S_FULL + i], 1);
            mbar_init(&bars[AB_P_FULL + i], 4);
            mbar_init(&bars[AB_PV_DONE + i], 1);
        }
        for (int i = 0; i < A_FBARS; ++i) {
            mbar_init(&bars[AB_K_FULL + i], 1);
            mbar_init(&bars[AB_V_FULL + i], 1);
        }
        for (int i = 0; i < A_KSLOTS; ++i) mbar_init(&bars[AB_K_EMPTY + i], 1);
        for (int i = 0; i < A_VSLOTS; ++i) mbar_init(&bars[AB_V_EMPTY + i], 1);
        fence_mbar_init();
        const bool plan_ok = ph.x == PLAN_MAGIC && ph.y == p.seq_len && ph.z == p.bm && ph.w == p.bn;
        if (!plan_ok && p.status != nullptr) atomicCAS(p.status, 0, STATUS_BAD_INDEX);
        *abort_flag = (st != 0 || !plan_ok) ? 1 : 0;
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, A_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (*abort_flag == 0) {
        if (warp == 4) {
            // -------------------------------------------------------------- TMA producer
            if (elect_one()) {
                tma_prefetch_desc(&map_q);
                tma_prefetch_desc(&map_q16);
                tma_prefetch_desc(&map_k);
                tma_prefetch_desc(&map_v);
                // two cursors over the block's stream of steps (steps of its items that have any): K loads run A_SBUF steps ahead
                // of the V loads, in the order the MMA warp consumes them.  `it` counts the items with steps (Q buffers alternate).
                // A step takes one ring slot when both halves work on the same tile (or one of them has none), else two: first
                // the tile of half A, then the tile of half B; all of a step's bytes are reported to the step's one barrier.
                // (the step word of a cursor's position is requested when the cursor gets there, a step before it is needed)
                struct Cursor { ItemQueue q; Item item; int j, it; uint32_t word; };
                auto settle = [&](Cursor& c) {
                    c.q.skip_empty(p, plan_sched);
                    c.item = c.q.cur;
                    if (c.item.valid) c.word = __ldg(plan_steps + static_cast<size_t>(c.item.qt) * p.max_steps);
                };
                auto advance = [&](Cursor& c) {
                    if (++c.j >= c.item.n) { c.j = 0; ++c.it; c.q.pop(p, plan_sched); settle(c); }
                    else c.word = __ldg(plan_steps + static_cast<size_t>(c.item.qt) * p.max_steps + c.j);
                };
                auto step_word = [&](const Cursor& c) { return c.word; };
                Cursor kc, vc;
                kc.q.init(p, plan_sched);
                kc.j = 0; kc.it = 0; kc.word = 0;
                settle(kc);
                vc = kc;
                unsigned uk = 0, uv = 0;                      // ring slots used so far
                unsigned gk = 0, gv = 0;                      // steps loaded so far
                auto load_k = [&]() {
                    if (kc.j == 0) {
                        const int qb = kc.it % A_QBUFS;
                        mbar_wait(&bars[AB_Q_EMPTY + qb], static_cast<uint32_t>(((kc.it / A_QBUFS) & 1) ^ 1), wctx, AB_Q_EMPTY + qb);
                        // the item's two 64-row halves (the second may be missing; its rows then carry "absent" codes only)
                        const int2 hr = __ldg(plan_halves + kc.item.qt);
                        unsigned char* qd = q_smem + qb * A_QBUF_BYTES;
                        uint64_t* qfull = &bars[AB_Q_FULL + qb];
                        mbar_arrive_expect_tx(qfull, hr.y >= 0 ? A_QBUF_BYTES : A_Q_BYTES / 2);
                        tma_tile(qd, &map_q, qfull, hr.x, kc.item.head, kc.item.batch, p.slot_s[0], p.slot_h[0], p.slot_b[0]);
                        if (hr.y >= 0) {
                            tma_tile(qd + A_Q_BYTES / 2, &map_q, qfull, hr.y, kc.item.head, kc.item.batch, p.slot_s[0], p.slot_h[0], p.slot_b[0]);
                            // the interleaved copy: 16-row boxes of half A and half B in turn
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                tma_tile(qd + A_Q_BYTES + (2 * c) * 2048, &map_q16, qfull, hr.x + 16 * c, kc.item.head, kc.item.batch, p.slot_s[0],
                                         p.slot_h[0], p.slot_b[0]);
                                tma_tile(qd + A_Q_BYTES + (2 * c + 1) * 2048, &map_q16, qfull, hr.y + 16 * c, kc.item.head, kc.item.batch, p.slot_s[0],
                                         p.slot_h[0], p.slot_b[0]);
                            }
                        }
                    }
                    const uint32_t w = step_word(kc);
                    const unsigned ta = w & 0xFFFFu, tb = w >> 16;
                    const unsigned first = ta != A_NO_TILE ? ta : tb;
                    const int tiles = (ta != A_NO_TILE && tb != A_NO_TILE && ta != tb) ? 2 : 1;
                    uint64_t* full = &bars[AB_K_FULL + gk % A_FBARS];
                    for (int i = 0; i < tiles; ++i, ++uk) {
                        const int sl = static_cast<int>(uk % A_KSLOTS);
                        mbar_wait(&bars[AB_K_EMPTY + sl], ((uk / A_KSLOTS) & 1) ^ 1, wctx, AB_K_EMPTY + sl);
                        if (i == 0) mbar_arrive_expect_tx(full, tiles * A_KV_BYTES);
                        tma_tile(k_smem + sl * A_KV_BYTES, &map_k, full, static_cast<int>(i == 0 ? first : tb) * A_TKV, kc.item.head,
                                 kc.item.batch, p.slot_s[1], p.slot_h[1], p.slot_b[1]);
                    }
                    ++gk;
                    advance(kc);
                };
                for (int i = 0; i < A_SBUF && kc.item.valid; ++i) load_k();
                while (vc.item.valid) {
                    const uint32_t w = step_word(vc);
                    const unsigned ta = w & 0xFFFFu, tb = w >> 16;
                    const unsigned first = ta != A_NO_TILE ? ta : tb;
                    const int tiles = (ta != A_NO_TILE && tb != A_NO_TILE && ta != tb) ? 2 : 1;
                    uint64_t* full = &bars[AB_V_FULL + gv % A_FBARS];
                    for (int i = 0; i < tiles; ++i, ++uv) {
                        const int sl = static_cast<int>(uv % A_VSLOTS);
                        mbar_wait(&bars[AB_V_EMPTY + sl], ((uv / A_VSLOTS) & 1) ^ 1, wctx, AB_V_EMPTY + sl);
                        if (i == 0) mbar_arrive_expect_tx(full, tiles * A_KV_BYTES);
                        tma_tile(v_smem + sl * A_KV_BYTES, &map_v, full, static_cast<int>(i == 0 ? first : tb) * A_TKV, vc.item.head,
                                 vc.item.batch, p.slot_s[2], p.slot_h[2], p.slot_b[2]);
                    }
                    ++gv;
                    advance(vc);
                    if (kc.item.valid) load_k();
                }
            }
        } else if (warp == 5) {
            // -------------------------------------------------------------- MMA issuer
            if (elect_one()) {
                constexpr uint32_t idesc_qk = make_idesc_f16(A_HALF, A_TKV, /*b_mn_major=*/false);
                constexpr uint32_t idesc_pv = make_idesc_f16(A_HALF, A_D, /*b_mn_major=*/true);
                constexpr uint32_t idesc_qk2 = make_idesc_f16(A_TQ, A_TKV, /*b_mn_major=*/false);     // both halves in one product
                constexpr uint32_t idesc_pv2 = make_idesc_f16(A_TQ, A_D, /*b_mn_major=*/true);
                // shared-memory descriptors of buffer 0 / slot 0; the others follow by adding their byte offset / 16
                const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(q_smem), 16, 1024);
                const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(k_smem), 16, 1024);
                const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(v_smem), 16, 1024);
                // two cursors over the same stream of steps: the QK^T cursor runs A_SBUF steps ahead of the PV cursor.  The step
                // word of a cursor's position is requested as soon as the cursor gets there, a whole step before it is needed.
                struct Cursor { ItemQueue q; int qt, n, j, it; bool valid; uint32_t word; };
                auto settle = [&](Cursor& c) {
                    c.q.skip_empty(p, plan_sched);
                    c.valid = c.q.cur.valid;
                    c.n = c.q.cur.n;
                    c.qt = c.q.cur.qt;
                    if (c.valid) c.word = __ldg(plan_steps + static_cast<size_t>(c.qt) * p.max_steps);
                };
                auto advance = [&](Cursor& c) {
                    if (++c.j >= c.n) { c.j = 0; ++c.it; c.q.pop(p, plan_sched); settle(c); }
                    else c.word = __ldg(plan_steps + static_cast<size_t>(c.qt) * p.max_steps + c.j);
                };
                Cursor qk, pv;
                qk.q.init(p, plan_sched);
                qk.j = 0; qk.it = 0; qk.word = 0;
                settle(qk);
                pv = qk;
                unsigned gq = 0, g = 0;                       // steps issued: QK^T, PV
                unsigned uq = 0, uv = 0;                      // ring slots consumed: K, V
                // S = Q K^T of step gq into buffer gq % A_SBUF, half A in lanes 0-15 of each quarter, half B in lanes 16-31.  The
                // buffer held S and P of step gq - A_SBUF: the PV products that read that P were issued before and the tensor core
                // executes this thread's MMAs in order.
                auto issue_qk = [&]() {
                    const int qb = qk.it % A_QBUFS;
                    if (qk.j == 0) mbar_wait(&bars[AB_Q_FULL + qb], static_cast<uint32_t>((qk.it / A_QBUFS) & 1), wctx, AB_Q_FULL + qb);
                    const uint32_t w = qk.word;
                    const unsigned ta = w & 0xFFFFu, tb = w >> 16;
                    const bool two = ta != A_NO_TILE && tb != A_NO_TILE && ta != tb;
                    const int sl0 = static_cast<int>(uq % A_KSLOTS), sl1 = static_cast<int>((uq + 1) % A_KSLOTS);
                    const int fb = static_cast<int>(gq % A_FBARS);
                    mbar_wait(&bars[AB_K_FULL + fb], (gq / A_FBARS) & 1, wctx, AB_K_FULL + fb);
                    tc_fence_after();
                    const uint64_t qd = q_desc0 + static_cast<uint64_t>(qb * (A_QBUF_BYTES >> 4));
                    const int sb = static_cast<int>(gq % A_SBUF);
                    const uint32_t d = tmem_base + A_COL_S + sb * A_TKV;
                    const uint64_t kd0 = k_desc0 + static_cast<uint64_t>(sl0 * (A_KV_BYTES >> 4));
                    if (ta == tb) {
                        mma_chain_qk(d, qd + (A_Q_BYTES >> 4), kd0, idesc_qk2);        // the interleaved rows: one M = 128 product chain
                    } else {
                        if (ta != A_NO_TILE) mma_chain_qk(d, qd, kd0, idesc_qk);
                        if (tb != A_NO_TILE)
                            mma_chain_qk(d + A_LANE_B, qd + (A_Q_BYTES >> 5), two ? k_desc0 + static_cast<uint64_t>(sl1 * (A_KV_BYTES >> 4)) : kd0, idesc_qk);
                    }
                    tc_commit(&bars[AB_K_EMPTY + sl0]);
                    if (two) tc_commit(&bars[AB_K_EMPTY + sl1]);
                    tc_commit(&bars[AB_S_FULL + sb]);
                    if (qk.j == qk.n - 1) tc_commit(&bars[AB_Q_EMPTY + qb]);     // every QK^T of that item has been issued
                    advance(qk);
                    ++gq;
                    uq += two ? 2u : 1u;
                };
                for (int i = 0; i < A_SBUF && qk.valid; ++i) issue_qk();
                while (pv.valid) {
                    if (pv.j == 0) mbar_wait(&bars[AB_O_FREE], static_cast<uint32_t>((pv.it & 1) ^ 1), wctx, AB_O_FREE);     // the previous item's O was read
                    const uint32_t o_tmem = tmem_base + A_COL_O;
                    const uint32_t w = pv.word;
                    const unsigned ta = w & 0xFFFFu, tb = w >> 16;
                    const bool two = ta != A_NO_TILE && tb != A_NO_TILE && ta != tb;
                    const int sb = static_cast<int>(g % A_SBUF);
                    const int sl0 = static_cast<int>(uv % A_VSLOTS), sl1 = static_cast<int>((uv + 1) % A_VSLOTS);
                    const int fb = static_cast<int>(g % A_FBARS);
                    mbar_wait(&bars[AB_V_FULL + fb], (g / A_FBARS) & 1, wctx, AB_V_FULL + fb);      // long there: off the P -> PV path
                    mbar_wait(&bars[AB_P_FULL + sb], (g / A_SBUF) & 1, wctx, AB_P_FULL + sb);
                    tc_fence_after();
                    const uint32_t p_tmem = tmem_base + A_COL_S + sb * A_TKV;
                    const uint32_t acc = pv.j > 0 ? 1u : 0u;
                    // a half's steps are the first ones of the item, so its first product (which overwrites O) comes at step 0
                    const uint64_t vd0 = v_desc0 + static_cast<uint64_t>(sl0 * (A_KV_BYTES >> 4));
                    if (ta == tb) {
                        mma_chain_pv(o_tmem, p_tmem, vd0, idesc_pv2, acc);
                    } else {
                        if (ta != A_NO_TILE) mma_chain_pv(o_tmem, p_tmem, vd0, idesc_pv, acc);
                        if (tb != A_NO_TILE)
                            mma_chain_pv(o_tmem + A_LANE_B, p_tmem + A_LANE_B,
                                         two ? v_desc0 + static_cast<uint64_t>(sl1 * (A_KV_BYTES >> 4)) : vd0, idesc_pv, acc);
                    }
                    tc_commit(&bars[AB_V_EMPTY + sl0]);
                    if (two) tc_commit(&bars[AB_V_EMPTY + sl1]);
                    tc_commit(&bars[AB_PV_DONE + sb]);
                    advance(pv);
                    ++g;
                    uv += two ? 2u : 1u;
                    if (qk.valid) issue_qk();                                     // into the buffer this PV has just been issued for
                }
            }
        } else {
            // -------------------------------------------------------------- softmax warps (one row per thread)
            // lanes 0-15 of the warp own rows 16 * warp .. + 15 of half A, lanes 16-31 the same rows of half B
            const int hsel = lane >> 4;                      // which half this thread's row belongs to
            const int rih = warp * 16 + (lane & 15);         // row inside the half
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
            const int rg = hsel * 4 + warp;                  // 16-row group of the plan codes
            const float scale = p.scale_log2, inv_scale = 1.0f / p.scale_log2;
            unsigned g = 0;                                  // steps of this block so far (matches the MMA warp's count)
            int sbuf = 0;                                    // g % A_SBUF and (g / A_SBUF) & 1, kept as running values
            uint32_t sphase = 0;
            // per-item values that need global loads are fetched one item ahead (no dependent-load chain at item boundaries)
            // first sequence row of the 64-row half this thread works on (-1: the item has no such half)
            auto item_half = [&](const Item& x) -> int {
                return x.valid ? __ldg(reinterpret_cast<const int*>(plan_halves) + 2 * x.qt + hsel) : -1;
            };
            auto item_row_base = [&](const Item& x, int half_row) -> int {
                const int r = half_row + rih;
                return (x.valid && x.n > 0 && half_row >= 0 && r < p.seq_len) ? __ldg(p.part_row_ptr + (r >> p.bm_shift)) : 0;
            };
            auto item_codes = [&](const Item& x) -> const uint2* {
                return reinterpret_cast<const uint2*>(plan_codes + (static_cast<size_t>(x.qt) * p.max_steps) * 32 + rg * 4);
            };
            unsigned char* slab = o_smem + warp * A_OSTAGE_BYTES;       // this warp's 32 x 128 B output staging (1024-aligned)
            // writes one fp16 output row (8 x 16 B) into the slab in the 128-byte-swizzled layout of the output tensor map
            // (slab rows 0-15: half A, 16-31: half B), then one lane per half hands its 16 rows to the TMA store; rows beyond the
            // sequence end are clipped by the tensor map
            auto store_rows = [&](const uint4 (&u)[8], const Item& x, int half_row) {
                if ((lane & 15) == 0) tma_store_wait_read();             // this lane's previous store has finished reading the slab
                __syncwarp();
#pragma unroll
                for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(slab + lane * 128 + ((c ^ (lane & 7)) << 4)) = u[c];
                fence_proxy_async_smem();
                __syncwarp();
                if ((lane & 15) == 0 && half_row >= 0) {
                    tma_tile_store(&map_o, slab + hsel * (A_OSTAGE_BYTES / 2), half_row + warp * 16, x.head, x.batch, p.slot_s[3], p.slot_h[3],
                                   p.slot_b[3]);
                    tma_store_commit();
                }
            };
            // item pipeline: what items k+1 and k+2 need from global memory (step count, half rows, row pointer, first codes:
            // chains of dependent loads) is requested while item k waits for its last PV product, and the schedule entry that
            // names item k+3 with it, so that decoding an item never waits for its number
            const ItemSource isrc = item_source(p);
            Item cur_item = fetch_item(0, isrc, p, plan_sched);
            Item item1 = fetch_item(1, isrc, p, plan_sched);
            unsigned id_ahead = fetch_item_id(2, isrc);      // number of item k + 2, requested an item before it is decoded
            int half_row = item_half(cur_item), half1 = item_half(item1);
            int part_base = item_row_base(cur_item, half_row);
            uint2 cw = (cur_item.valid && cur_item.n > 0) ? __ldg(item_codes(cur_item)) : make_uint2(0u, 0u);      // codes of step 0
            for (unsigned k = 0; cur_item.valid; ++k) {
                // the values of the items after this one; they replace the current ones at the end of the iteration
                Item item2;
                int half2, part_base1;
                uint2 cw1;
                auto fetch_ahead = [&]() {
                    part_base1 = item_row_base(item1, half1);
                    cw1 = (item1.valid && item1.n > 0) ? __ldg(item_codes(item1)) : make_uint2(0u, 0u);
                    item2 = decode_item(id_ahead, p, plan_sched);
                    id_ahead = fetch_item_id(k + 3, isrc);
                    half2 = item_half(item2);
                };
                auto rotate = [&]() {
                    cur_item = item1; half_row = half1; part_base = part_base1; cw = cw1;
                    item1 = item2; half1 = half2;
                };
                const int n = cur_item.n;
                if (n == 0) {
                    uint4 z[8];
#pragma unroll
                    for (int c = 0; c < 8; ++c) z[c] = make_uint4(0u, 0u, 0u, 0u);
                    store_rows(z, cur_item, half_row);
                    fetch_ahead();
                    rotate();
                    continue;
                }
                const uint2* my_codes = item_codes(cur_item);
                float m_ref = -INFINITY, l_sum = 0.f;

                for (int j = 0; j < n; ++j, ++g) {
                    const int b = sbuf;
                    const uint32_t bphase = sphase;
                    if (++sbuf == A_SBUF) { sbuf = 0; sphase ^= 1u; }
                    const uint2 cur = cw;
                    if (j + 1 < n) cw = __ldg(my_codes + (j + 1) * 8);     // 32 codes = 64 B = 8 uint2 per step
                    // class of this warp's 32 x 64 part of the step, put into the codes by the plan: the same value in every lane
                    const unsigned warp_class = cur.y >> 30;
                    const bool warp_absent = warp_class == 0u, warp_fast = warp_class == 1u;
                    // a thread whose 16-row group lists nothing of this step keeps its maximum and its sum: either its half has no
                    // tile at this step (no product was issued for it: the scores it loads are stale and what it computes from
                    // them is never used) or its scores were all set to -inf by the masking (P = 0)
                    const bool present = (cur.x | (cur.y & 0x3FFFFFFFu)) != 0u;
                    mbar_wait(&bars[AB_S_FULL + b], bphase, wctx, AB_S_FULL + b);
                    tc_fence_after();
                    uint32_t r0[32], r1[32];
                    if (warp_absent) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) r0[i] = 0u;
                    } else {
                        if (!warp_fast)
                            mask_scores_in_tmem(t_lane + A_COL_S + b * A_TKV, cur.x, cur.y, p.part_block_mask, part_base, p.bm_shift, p.bn,
                                                (half_row + rih) & (p.bm - 1),
                                                static_cast<int>((__ldg(plan_steps + static_cast<size_t>(cur_item.qt) * p.max_steps + j) >> (16 * hsel)) & 0xFFFFu) * A_TKV);
                        tmem_ld32(t_lane + A_COL_S + b * A_TKV, r0);
                        tmem_ld32(t_lane + A_COL_S + b * A_TKV + 32, r1);
                        tc_wait_ld();
                        // row maximum of the raw scores (four independent chains of 3-input maxima), then in log2 units
                        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            mx0 = max3(mx0, __uint_as_float(r0[i]), __uint_as_float(r1[i]));
                            mx1 = max3(mx1, __uint_as_float(r0[i + 1]), __uint_as_float(r1[i + 1]));
                            mx2 = max3(mx2, __uint_as_float(r0[i + 2]), __uint_as_float(r1[i + 2]));
                            mx3 = max3(mx3, __uint_as_float(r0[i + 3]), __uint_as_float(r1[i + 3]));
                        }
                        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale;
                        // lazy rescale: move the reference maximum only when it would grow by more than the threshold
                        const bool need = present && (mx > m_ref + A_RESCALE_THRESHOLD || (m_ref == -INFINITY && mx > -INFINITY));
                        if (__any_sync(0xffffffffu, need)) {
                            float alpha = 1.0f;
                            if (need) {
                                // the reference is kept integer-valued (the polynomial exponential folds it into its rounding constant)
                                const float m_new = fminf(fmaxf(ceilf(mx), -2097152.0f), 2097152.0f);
                                alpha = (m_ref == -INFINITY) ? 0.0f : fast_exp2(m_ref - m_new);
                                m_ref = m_new;
                                l_sum *= alpha;
                            }
                            if (j > 0) {
                                // every PV product issued so far for this item must have landed in O before it is rescaled
                                const int pb = static_cast<int>((g - 1) % A_SBUF);
                                mbar_wait(&bars[AB_PV_DONE + pb], ((g - 1) / A_SBUF) & 1, wctx, AB_PV_DONE + pb);
                                tc_fence_after();
                                rescale_o_in_tmem(t_lane + A_COL_O, alpha);
                            }
                        }
                        // P = 2^(s * scale - m) for the 64 scores in r0/r1: pairs of columns with packed fp32 FMAs; A_POLY_PAIRS of
                        // every 8 pairs take the FMA-pipe polynomial instead of the MUFU unit.  The fp16 pairs of P are written over
                        // r0 as its scores are consumed.
                        const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref;
                        const float2 scale2 = pk2(scale, scale), negm2 = pk2(neg_m, neg_m);
                        const float2 mm2 = pk2(12582912.0f + neg_m, 12582912.0f + neg_m);
                        const float lo = (-120.0f - neg_m) * inv_scale;
                        float2 sum_a = pk2(0.f, 0.f), sum_b = pk2(0.f, 0.f);
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float s0 = __uint_as_float((i < 16) ? r0[2 * i] : r1[2 * (i - 16)]);
                            const float s1 = __uint_as_float((i < 16) ? r0[2 * i + 1] : r1[2 * (i - 16) + 1]);
                            float e0, e1;
                            if (((i * A_POLY_PAIRS) & 7) < A_POLY_PAIRS) {         // A_POLY_PAIRS of every 8 pairs, evenly spread
                                exp2_poly_pair(s0, s1, lo, scale2, mm2, e0, e1);
                            } else {
                                float x0, x1;
                                upk2(fma2(pk2(s0, s1), scale2, negm2), x0, x1);
                                e0 = fast_exp2(x0);
                                e1 = fast_exp2(x1);
                            }
                            if (i & 1) sum_b = add2(sum_b, pk2(e0, e1));
                            else sum_a = add2(sum_a, pk2(e0, e1));
                            r0[i] = pack_half2(e0, e1);          // pair i of P; r0[2i], r0[2i+1] were consumed above
                        }
                        float sa0, sa1;
                        upk2(add2(sum_a, sum_b), sa0, sa1);
                        if (present) l_sum += sa0 + sa1;
                    }
                    // P overlays the first 32 columns of the S buffer it was computed from; the QK^T that next writes this
                    // buffer is issued after the PV products that read P and the tensor core executes them in that order
                    tmem_st32(t_lane + A_COL_S + b * A_TKV, r0);
                    tc_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars[AB_P_FULL + b]);
                }
                // ---------------------------------------------------------- item epilogue: O / l -> fp16 -> global
                fetch_ahead();                                  // the loads for the next items overlap the wait for the last PV product
                {
                    const int pb = static_cast<int>((g - 1) % A_SBUF);
                    mbar_wait(&bars[AB_PV_DONE + pb], ((g - 1) / A_SBUF) & 1, wctx, AB_PV_DONE + pb);
                    tc_fence_after();
                    uint32_t o0[32], o1[32];
                    tmem_ld32(t_lane + A_COL_O, o0);
                    tmem_ld32(t_lane + A_COL_O + 32, o1);
                    tc_wait_ld();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars[AB_O_FREE]);
                    {
                        // a row that accumulated nothing (no listed key, or a half without any step: its O was never written) gives zeros
                        const bool any = l_sum > 0.f;
                        const float inv = any ? 1.0f / l_sum : 0.0f;
                        uint4 u[8];
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const uint32_t* src = (c < 4) ? &o0[c * 8] : &o1[(c - 4) * 8];
                            u[c].x = any ? pack_half2(__uint_as_float(src[0]) * inv, __uint_as_float(src[1]) * inv) : 0u;
                            u[c].y = any ? pack_half2(__uint_as_float(src[2]) * inv, __uint_as_float(src[3]) * inv) : 0u;
                            u[c].z = any ? pack_half2(__uint_as_float(src[4]) * inv, __uint_as_float(src[5]) * inv) : 0u;
                            u[c].w = any ? pack_half2(__uint_as_float(src[6]) * inv, __uint_as_float(src[7]) * inv) : 0u;
                        }
                        store_rows(u, cur_item, half_row);
                    }
                }
                rotate();
            }
            if ((lane & 15) == 0) tma_store_wait_all();      // every output store of this warp has been performed
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, A_TMEM_COLS);
    }
}

constexpr size_t A_SMEM_BYTES = 1024 + A_QBUFS * A_QBUF_BYTES + static_cast<size_t>(A_KSLOTS + A_VSLOTS) * A_KV_BYTES + 4 * A_OSTAGE_BYTES + AB_COUNT * 8 + 16;

// Sorts the three outer dimensions (row, head, batch) by stride so that the tensor map's strides ascend;
// returns the coordinate slot of each logical dimension.
int make_qkv_map(CUtensorMap* map, const void* base, int batch, int heads, int seq_len, const long long st[3], int box_rows, int* slot_s,
                 int* slot_h, int* slot_b) {
    struct Dim { uint64_t size; long long stride; int logical; } d[3] = {
        {static_cast<uint64_t>(seq_len), st[2], 0}, {static_cast<uint64_t>(heads), st[1], 1}, {static_cast<uint64_t>(batch), st[0], 2}};
    for (int i = 0; i < 3; ++i)
        for (int j = i + 1; j < 3; ++j)
            if (d[j].stride < d[i].stride) { Dim t = d[i]; d[i] = d[j]; d[j] = t; }
    uint64_t dims[4] = {A_D, 0, 0, 0}, strides[3];
    uint32_t box[4] = {A_D, 1, 1, 1};
    for (int i = 0; i < 3; ++i) {
        dims[i + 1] = d[i].size;
        strides[i] = static_cast<uint64_t>(d[i].stride) * 2;
        if (d[i].logical == 0) { box[i + 1] = static_cast<uint32_t>(box_rows); *slot_s = i + 1; }
        if (d[i].logical == 1) *slot_h = i + 1;
        if (d[i].logical == 2) *slot_b = i + 1;
    }
    return make_tensor_map_f16(map, base, 4, dims, strides, box);
}

int log2_exact(int v) {
    int s = 0;
    while ((1 << s) < v) ++s;
    return s;
}

// shared memory of the plan kernel: one 16-bit code per (row block of either half, column block), then three lists of key tiles
size_t plan_table_bytes(int seq_len, int block_m, int block_n) {
    return static_cast<size_t>(2 * (block_m >= 64 ? 1 : 64 / block_m)) * (seq_len / block_n) * 2 + 3 * static_cast<size_t>((seq_len + A_TKV - 1) / A_TKV) * 2;
}

int check_blocks(int seq_len, int block_m, int block_n) {
    STOF_REQUIRE(seq_len > 0, "block_attn: bad seq_len");
    STOF_REQUIRE(block_m == 16 || block_m == 32 || block_m == 64 || block_m == 128, "block_attn: BLOCK_M %d not in {16,32,64,128}", block_m);
    STOF_REQUIRE(block_n == 16 || block_n == 32 || block_n == 64 || block_n == 128, "block_attn: BLOCK_N %d not in {16,32,64,128}", block_n);
    STOF_REQUIRE(seq_len % block_m == 0 && seq_len % block_n == 0, "block_attn: seq_len %d not a multiple of BLOCK_M %d / BLOCK_N %d", seq_len,
                 block_m, block_n);
    const size_t table_bytes = plan_table_bytes(seq_len, block_m, block_n);
    if (table_bytes > A_MAX_TABLE_BYTES) {
        set_error("block_attn: seq_len %d with %dx%d blocks needs a %zu-byte block table, beyond the maximum of %d", seq_len, block_m, block_n,
                  table_bytes, A_MAX_TABLE_BYTES);
        return STOF_E_LIMIT;
    }
    return STOF_OK;
}

}  // namespace
}  // namespace stof

using namespace stof;


extern "C" size_t stof_block_attn_plan_bytes(int seq_len, int block_m, int block_n) {
    if (seq_len <= 0 || block_m <= 0 || block_n <= 0) return 0;
    const int nqt = (seq_len + A_TQ - 1) / A_TQ, maxt = (seq_len + A_TKV - 1) / A_TKV;
    return plan_total_bytes(nqt, maxt) + 16;          // trailing 16 bytes: the ticket of the plan kernel
}

static int launch_plan(const int* full_row_ptr, const int* full_col_idx, const int* part_row_ptr, const int* part_col_idx, const int* pairs,
                       int seq_len, int block_m, int block_n, void* plan, size_t plan_bytes, int* status_dev, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (int rc = check_blocks(seq_len, block_m, block_n)) return rc;
    STOF_REQUIRE(full_row_ptr && part_row_ptr && plan, "block_attn_plan: null pointer");
    STOF_REQUIRE(aligned16(plan), "block_attn_plan: plan buffer must be 16-byte aligned");
    const size_t need = stof_block_attn_plan_bytes(seq_len, block_m, block_n);
    if (plan_bytes < need) {
        set_error("block_attn_plan: plan buffer of %zu bytes, need %zu", plan_bytes, need);
        return STOF_E_WORKSPACE;
    }
    const int nqt = (seq_len + A_TQ - 1) / A_TQ, maxt = (seq_len + A_TKV - 1) / A_TKV;
    unsigned char* pl = static_cast<unsigned char*>(plan);
    unsigned int* ticket = reinterpret_cast<unsigned int*>(pl + plan_total_bytes(nqt, maxt));
    STOF_CUDA(cudaMemsetAsync(pl, 0, sizeof(PlanHeader), stream));
    STOF_CUDA(cudaMemsetAsync(ticket, 0, 16, stream));
    const size_t smem = plan_table_bytes(seq_len, block_m, block_n);
    static std::atomic<bool> configured[64];     // per device; host threads may race here, every one of them stores the same value
    int dev = 0;
    STOF_CUDA(cudaGetDevice(&dev));
    if (smem > 40 * 1024 && (dev < 0 || dev >= 64 || !configured[dev])) {
        STOF_CUDA(cudaFuncSetAttribute(plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A_MAX_TABLE_BYTES));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    plan_kernel<<<nqt, 256, smem, stream>>>(full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, reinterpret_cast<const int2*>(pairs), seq_len,
                                            block_m, block_n, pl, ticket, status_dev);
    STOF_CUDA(cudaGetLastError());
    return STOF_OK;
}

extern "C" int stof_block_attn_plan(const int* full_row_ptr, const int* full_col_idx, const int* part_row_ptr, const int* part_col_idx,
                                    int seq_len, int block_m, int block_n, void* plan, size_t plan_bytes, int* status_dev, void* stream) {
    return launch_plan(full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, nullptr, seq_len, block_m, block_n, plan, plan_bytes, status_dev,
                       stream);
}

extern "C" int stof_block_attn_plan_paired(const int* full_row_ptr, const int* full_col_idx, const int* part_row_ptr, const int* part_col_idx,
                                           const int* pairs, int seq_len, int block_m, int block_n, void* plan, size_t plan_bytes,
                                           int* status_dev, void* stream) {
    STOF_REQUIRE(pairs != nullptr, "block_attn_plan_paired: null pairs");
    STOF_REQUIRE((reinterpret_cast<uintptr_t>(pairs) & 7u) == 0, "block_attn_plan_paired: pairs must be 8-byte aligned");
    return launch_plan(full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, pairs, seq_len, block_m, block_n, plan, plan_bytes, status_dev,
                       stream);
}

static int launch_block_attn(const void* q, const void* k, const void* v, void* out, int batch, int heads, int seq_len, int head_dim,
                             const long long q_strides[3], const long long k_strides[3], const long long v_strides[3],
                             const long long out_strides[3], const int* part_row_ptr, const void* part_block_mask, const void* plan,
                             int block_m, int block_n, int num_warps, float softmax_scale, const int* schedule, int schedule_blocks,
                             int* status_dev, void* stream_) {
    (void)num_warps;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    STOF_REQUIRE(q && k && v && out, "block_attn: null q/k/v/out");
    STOF_REQUIRE(part_row_ptr && plan, "block_attn: null part_row_ptr or plan");
    STOF_REQUIRE(head_dim == A_D, "block_attn: head_dim %d unsupported (the kernels are built for 64, as the reference's are)", head_dim);
    STOF_REQUIRE(batch > 0 && heads > 0, "block_attn: bad shape");
    if (int rc = check_blocks(seq_len, block_m, block_n)) return rc;
    STOF_REQUIRE(softmax_scale > 0.f, "block_attn: softmax_scale must be positive");
    STOF_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(part_block_mask) && aligned16(plan),
                 "block_attn: pointers must be 16-byte aligned");
    const long long* all[4] = {q_strides, k_strides, v_strides, out_strides};
    for (int t = 0; t < 4; ++t) {
        STOF_REQUIRE(all[t] != nullptr, "block_attn: null stride array");
        for (int i = 0; i < 3; ++i)
            STOF_REQUIRE(all[t][i] > 0 && all[t][i] % 8 == 0, "block_attn: strides must be positive multiples of 8 elements");
    }
    AttnParams p;
    p.part_row_ptr = part_row_ptr;
    p.part_block_mask = static_cast<const __half*>(part_block_mask);
    p.plan = static_cast<const unsigned char*>(plan);
    p.batch = batch; p.heads = heads; p.seq_len = seq_len; p.bm = block_m; p.bn = block_n;
    p.bm_shift = log2_exact(block_m); p.bn_shift = log2_exact(block_n);
    p.n_qtiles = (seq_len + A_TQ - 1) / A_TQ;
    p.max_steps = (seq_len + A_TKV - 1) / A_TKV;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.status = status_dev;
    p.schedule = schedule;
    const long long items = static_cast<long long>(batch) * heads * p.n_qtiles;
    STOF_REQUIRE(items < (1ll << 31), "block_attn: batch * heads * query tiles beyond 2^31");
    p.total_items = static_cast<unsigned>(items);
    p.bh_total = static_cast<unsigned>(batch) * static_cast<unsigned>(heads);
    CUtensorMap mq, mq16, mk, mv, mo;
    int unused_slot[3];
    if (int rc = make_qkv_map(&mo, out, batch, heads, seq_len, out_strides, 16, &p.slot_s[3], &p.slot_h[3], &p.slot_b[3])) return rc;
    if (int rc = make_qkv_map(&mq, q, batch, heads, seq_len, q_strides, A_TQ / 2, &p.slot_s[0], &p.slot_h[0], &p.slot_b[0])) return rc;
    if (int rc = make_qkv_map(&mq16, q, batch, heads, seq_len, q_strides, 16, &unused_slot[0], &unused_slot[1], &unused_slot[2])) return rc;
    if (int rc = make_qkv_map(&mk, k, batch, heads, seq_len, k_strides, A_TKV, &p.slot_s[1], &p.slot_h[1], &p.slot_b[1])) return rc;
    if (int rc = make_qkv_map(&mv, v, batch, heads, seq_len, v_strides, A_TKV, &p.slot_s[2], &p.slot_h[2], &p.slot_b[2])) return rc;

    static std::atomic<bool> configured[64];     // per device; host threads may race here, every one of them stores the same value
    int dev = 0;
    STOF_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        STOF_CUDA(cudaFuncSetAttribute(block_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(A_SMEM_BYTES)));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    long long grid = static_cast<long long>(A_CTAS_PER_SM) * sm_count();
    if (grid > items) grid = items;
    if (schedule != nullptr) {
        // every block of the table must be resident at once (the kernel is persistent: one block per table entry)
        STOF_REQUIRE(schedule_blocks >= 1 && schedule_blocks <= A_CTAS_PER_SM * sm_count(),
                     "block_attn: schedule made for %d thread blocks, this GPU runs at most %d", schedule_blocks, A_CTAS_PER_SM * sm_count());
        STOF_REQUIRE((reinterpret_cast<uintptr_t>(schedule) & 3u) == 0, "block_attn: schedule must be 4-byte aligned");
        grid = schedule_blocks;
    }
    block_attn_kernel<<<static_cast<unsigned>(grid), A_THREADS, A_SMEM_BYTES, stream>>>(mq, mq16, mk, mv, mo, p);
    STOF_CUDA(cudaGetLastError());
    return STOF_OK;
}

extern "C" int stof_block_attn(const void* q, const void* k, const void* v, void* out, int batch, int heads, int seq_len, int head_dim,
                               const long long q_strides[3], const long long k_strides[3], const long long v_strides[3],
                               const long long out_strides[3], const int* part_row_ptr, const void* part_block_mask, const void* plan,
                               int block_m, int block_n, int num_warps, float softmax_scale, int* status_dev, void* stream) {
    return launch_block_attn(q, k, v, out, batch, heads, seq_len, head_dim, q_strides, k_strides, v_strides, out_strides, part_row_ptr,
                             part_block_mask, plan, block_m, block_n, num_warps, softmax_scale, nullptr, 0, status_dev, stream);
}

extern "C" int stof_block_attn_scheduled(const void* q, const void* k, const void* v, void* out, int batch, int heads, int seq_len,
                                         int head_dim, const long long q_strides[3], const long long k_strides[3],
                                         const long long v_strides[3], const long long out_strides[3], const int* part_row_ptr,
                                         const void* part_block_mask, const void* plan, int block_m, int block_n, int num_warps,
                                         float softmax_scale, const int* schedule, int schedule_blocks, int* status_dev, void* stream) {
    STOF_REQUIRE(schedule != nullptr, "block_attn_scheduled: null schedule");
    return launch_block_attn(q, k, v, out, batch, heads, seq_len, head_dim, q_strides, k_strides, v_strides, out_strides, part_row_ptr,
                             part_block_mask, plan, block_m, block_n, num_warps, softmax_scale, schedule, schedule_blocks, status_dev, stream);
}
