// Mask -> block-CSR index compaction (integer, bit-exact, HBM-bound).
//
// Semantics follow get_sparse_storage of the reference (src/util/masks.py:125-184): tiles of mask[0]
// are scanned row-major; a tile whose elements all equal 1 is "full", all equal 0 "empty", anything
// else "partial" and carries the fp16 tile -10000 * (1 - m).  `load` merges full and partial in
// column order.  The element count of non-zeros runs over the whole (batch, S, S) tensor.
//
// Phase 1 (classify_kernel): the mask is streamed once with 128-bit loads.  A thread block owns a
// stripe of one block-row by a run of whole tiles, keeps two byte flags per tile in shared memory
// (saw-a-non-one / saw-a-non-zero) and writes one class byte per tile.  The last block to finish
// (atomic ticket) turns the class bytes into per-row counts (independent loads + shared-memory atomics) and into the three
// row-pointer arrays with a warp-shuffle prefix sum.
// Phase 2 (fill_kernel): one warp per block-row ranks its tiles with ballots + popc to place the
// column indices; the partial tiles of the row are then gathered by the whole thread block.
#include "stof_host.h"

#include <cuda_fp16.h>

#include <mutex>

namespace stof {
namespace {

constexpr int CLS_EMPTY = 0;
constexpr int CLS_FULL = 1;
constexpr int CLS_PART = 2;

constexpr int CLASSIFY_THREADS = 256;
constexpr int MAX_TILES_PER_STRIPE = 4096;
constexpr int FILL_THREADS = 256;

struct Workspace {            // header at the start of the caller's workspace, class bytes follow
    unsigned int ticket;      // blocks that finished phase 1 (reset by the last one)
    unsigned int pad[3];
};
constexpr size_t WS_HEADER = 16;

__host__ __device__ inline size_t cls_bytes(int nbm, int nbn) { return (static_cast<size_t>(nbm) * nbn + 15) & ~static_cast<size_t>(15); }

// flags for one 16-byte chunk: bit0 = some element != 1, bit1 = some element != 0; also the non-zero count.
// Masks are made of runs of equal values, so nearly every chunk is eight ones or eight zeros: both cases are settled on the
// whole chunk with a handful of word operations (AND / OR of the four words against the bit pattern of 1.0, sign bits ignored
// for zero: -0.0 == 0), and only a mixed chunk is looked at element by element.
template <bool F32>
__device__ __forceinline__ void chunk_flags(const uint4& v, unsigned& flags, unsigned& nz) {
    constexpr unsigned ONE = F32 ? 0x3F800000u : 0x3C003C00u;
    constexpr unsigned MAG = F32 ? 0x7FFFFFFFu : 0x7FFF7FFFu;
    const unsigned all_and = v.x & v.y & v.z & v.w, all_or = v.x | v.y | v.z | v.w;
    if (all_and == ONE && all_or == ONE) {                 // every element is exactly 1.0
        flags |= 2u;
        nz += F32 ? 4u : 8u;
        return;
    }
    if ((all_or & MAG) == 0u) {                            // every element is +0.0 or -0.0
        flags |= 1u;
        return;
    }
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
    if (F32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const bool zero = (w[i] & 0x7FFFFFFFu) == 0u;
            flags |= (w[i] != 0x3F800000u ? 1u : 0u) | (zero ? 0u : 2u);
            nz += zero ? 0u : 1u;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const unsigned lo = w[i] & 0xFFFFu, hi = w[i] >> 16;
            const bool zlo = (lo & 0x7FFFu) == 0u, zhi = (hi & 0x7FFFu) == 0u;
            flags |= ((lo != 0x3C00u || hi != 0x3C00u) ? 1u : 0u) | ((zlo && zhi) ? 0u : 2u);
            nz += (zlo ? 0u : 1u) + (zhi ? 0u : 1u);
        }
    }
}

// Runs in the last block of phase 1: class bytes -> row counts -> row pointers and totals.
__device__ void scan_rows(const unsigned char* cls, int nbm, int nbn, int* full_row_ptr, int* part_row_ptr, int* load_row_ptr,
                          unsigned long long* counts, int* row_counts /* smem, 2 * nbm_chunk */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int carry_full = 0, carry_part = 0;
    if (threadIdx.x == 0) {
        full_row_ptr[0] = 0;
        part_row_ptr[0] = 0;
        load_row_ptr[0] = 0;
    }
    // rows are processed in chunks of 32 * nwarps: every thread loads class bytes of the chunk independently
    // (no serial chain of dependent loads) and counts into shared memory, then warp 0 scans the chunk
    const int chunk = 32 * nwarps;
    for (int r0 = 0; r0 < nbm; r0 += chunk) {
        for (int i = threadIdx.x; i < 2 * chunk; i += blockDim.x) row_counts[i] = 0;
        __syncthreads();
        const int rows_here = min(chunk, nbm - r0);
        const long long cells = static_cast<long long>(rows_here) * nbn;
        for (long long i = threadIdx.x; i < cells; i += blockDim.x) {
            const int k = __ldcg(cls + static_cast<size_t>(r0) * nbn + i);
            if (k != CLS_EMPTY) atomicAdd(&row_counts[2 * static_cast<int>(i / nbn) + (k == CLS_PART ? 1 : 0)], 1);
        }
        __syncthreads();
        if (warp == 0) {
            for (int g = 0; g < nwarps; ++g) {
                const int r = r0 + g * 32 + lane;
                int nf = r < nbm ? row_counts[2 * (g * 32 + lane)] : 0;
                int np = r < nbm ? row_counts[2 * (g * 32 + lane) + 1] : 0;
                int sf = nf, sp = np;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int tf = __shfl_up_sync(0xffffffffu, sf, o);
                    const int tp = __shfl_up_sync(0xffffffffu, sp, o);
                    if (lane >= o) {
                        sf += tf;
                        sp += tp;
                    }
                }
                if (r < nbm) {
                    full_row_ptr[r + 1] = carry_full + sf;
                    part_row_ptr[r + 1] = carry_part + sp;
                    load_row_ptr[r + 1] = carry_full + sf + carry_part + sp;
                }
                carry_full += __shfl_sync(0xffffffffu, sf, 31);
                carry_part += __shfl_sync(0xffffffffu, sp, 31);
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        counts[0] = static_cast<unsigned long long>(carry_full);
        counts[1] = static_cast<unsigned long long>(carry_part);
        counts[2] = static_cast<unsigned long long>(carry_full + carry_part);
    }
}

template <bool F32>
__global__ void __launch_bounds__(CLASSIFY_THREADS)
classify_kernel(const void* __restrict__ mask, int seq_len, int bm, int bn, int stripe_cols, int* full_row_ptr, int* part_row_ptr,
                int* load_row_ptr, unsigned long long* counts, Workspace* ws, unsigned char* cls) {
    constexpr int EPC = F32 ? 4 : 8;                       // elements per 16-byte chunk
    __shared__ __align__(16) unsigned char s_flags[MAX_TILES_PER_STRIPE];
    __shared__ unsigned int s_nz[CLASSIFY_THREADS / 32];
    __shared__ int s_rows[2 * CLASSIFY_THREADS];
    __shared__ bool s_last;

    const int nbn = seq_len / bn, nbm = seq_len / bm;
    const int brow = blockIdx.y, batch = blockIdx.z;
    const int col0 = blockIdx.x * stripe_cols;
    const int cols = min(stripe_cols, seq_len - col0);
    const int tiles = cols / bn;
    for (int i = threadIdx.x; i < tiles; i += blockDim.x) s_flags[i] = 0;
    __syncthreads();

    const size_t elem_bytes = F32 ? 4 : 2;
    const char* base = static_cast<const char*>(mask) +
                       (static_cast<size_t>(batch) * seq_len * seq_len + static_cast<size_t>(brow) * bm * seq_len + col0) * elem_bytes;
    const int chunks_per_row = cols / EPC;
    const int total = bm * chunks_per_row;
    unsigned nz = 0;
    // four independent 16-byte loads in flight per thread before any of them is consumed.  Chunk idx of the block's
    // bm x chunks_per_row grid lies at (row, chunk) = (idx / chunks_per_row, idx % chunks_per_row); the four positions of a
    // thread advance by a fixed (rows, chunks) step per iteration, so the division is done once, outside the loop.
    constexpr int BATCH = 4;
    const int step = BATCH * blockDim.x;
    const int step_r = step / chunks_per_row, step_c = step - step_r * chunks_per_row;
    int pr[BATCH], pc[BATCH];
#pragma unroll
    for (int u = 0; u < BATCH; ++u) {
        const int idx = threadIdx.x + u * blockDim.x;
        pr[u] = idx / chunks_per_row;
        pc[u] = idx - pr[u] * chunks_per_row;
    }
    for (int idx0 = threadIdx.x; idx0 < total; idx0 += step) {
        uint4 v[BATCH];
        int tile_of[BATCH];
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            if (idx0 + u * static_cast<int>(blockDim.x) < total) {
                v[u] = __ldg(reinterpret_cast<const uint4*>(base + (static_cast<size_t>(pr[u]) * seq_len + pc[u] * EPC) * elem_bytes));
                tile_of[u] = (pc[u] * EPC) / bn;
            } else {
                tile_of[u] = -1;
            }
            pr[u] += step_r;
            pc[u] += step_c;
            if (pc[u] >= chunks_per_row) { pc[u] -= chunks_per_row; ++pr[u]; }
        }
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            if (tile_of[u] < 0) continue;
            unsigned f = 0;
            chunk_flags<F32>(v[u], f, nz);
            if (batch == 0 && f) {
                const int t = tile_of[u];
                // several threads may set the same bits; every writer ORs in bits that stay set
                if ((s_flags[t] & f) != f) atomicOr(reinterpret_cast<unsigned int*>(&s_flags[t & ~3]), f << (8 * (t & 3)));
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) nz += __shfl_xor_sync(0xffffffffu, nz, o);
    if ((threadIdx.x & 31) == 0) s_nz[threadIdx.x >> 5] = nz;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
        for (int i = 0; i < CLASSIFY_THREADS / 32; ++i) t += s_nz[i];
        if (t) atomicAdd(&counts[3], t);
    }
    if (batch == 0) {
        const int tile0 = col0 / bn;
        for (int i = threadIdx.x; i < tiles; i += blockDim.x) {
            const unsigned f = s_flags[i];
            cls[static_cast<size_t>(brow) * nbn + tile0 + i] =
                static_cast<unsigned char>((f & 1u) == 0u ? CLS_FULL : ((f & 2u) == 0u ? CLS_EMPTY : CLS_PART));
        }
    }
    // last block of the whole grid builds the row pointers
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned total_blocks = gridDim.x * gridDim.y * gridDim.z;
        const unsigned t = atomicAdd(&ws->ticket, 1u);
        s_last = (t == total_blocks - 1);
        if (s_last) ws->ticket = 0;                        // ready for the next call
    }
    __syncthreads();
    if (s_last) {
        __threadfence();
        scan_rows(cls, nbm, nbn, full_row_ptr, part_row_ptr, load_row_ptr, counts, s_rows);
    }
}

template <bool F32>
__global__ void __launch_bounds__(FILL_THREADS)
fill_kernel(const void* __restrict__ mask, int seq_len, int bm, int bn, const unsigned char* __restrict__ cls,
            const int* __restrict__ full_row_ptr, const int* __restrict__ part_row_ptr, const int* __restrict__ load_row_ptr,
            int* full_col_idx, int* part_col_idx, int* load_col_idx, __half* part_block_mask) {
    extern __shared__ int s_part_cols[];                   // columns of this row's partial tiles, nbn entries at most
    const int nbn = seq_len / bn;
    const int brow = blockIdx.x, share = blockIdx.y, shares = gridDim.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int f0 = full_row_ptr[brow], p0 = part_row_ptr[brow], l0 = load_row_ptr[brow];
    const int n_part = part_row_ptr[brow + 1] - p0;

    if (warp == 0) {
        int nf = 0, np = 0;
        for (int c0 = 0; c0 < nbn; c0 += 32) {
            const int c = c0 + lane;
            const int k = c < nbn ? cls[static_cast<size_t>(brow) * nbn + c] : CLS_EMPTY;
            const unsigned bf = __ballot_sync(0xffffffffu, k == CLS_FULL);
            const unsigned bp = __ballot_sync(0xffffffffu, k == CLS_PART);
            const unsigned lt = (1u << lane) - 1u;
            const int rf = nf + __popc(bf & lt), rp = np + __popc(bp & lt);
            if (k == CLS_FULL) {
                if (share == 0) {
                    full_col_idx[f0 + rf] = c;
                    load_col_idx[l0 + rf + rp] = c;
                }
            } else if (k == CLS_PART) {
                s_part_cols[rp] = c;
                if (share == 0) {
                    part_col_idx[p0 + rp] = c;
                    load_col_idx[l0 + rf + rp] = c;
                }
            }
            nf += __popc(bf);
            np += __popc(bp);
        }
    }
    __syncthreads();
    if (n_part == 0 || part_block_mask == nullptr) return;

    // gather: tile p of this row -> part_block_mask[p0 + p] = -10000 * (1 - m), 8 elements per thread step
    const int chunks_per_tile_row = bn / 8;
    const int chunks_per_tile = bm * chunks_per_tile_row;
    const __half one = __float2half(1.0f), neg = __float2half(-10000.0f);
    for (int p = share; p < n_part; p += shares) {
        const int c = s_part_cols[p];
        __half* dst = part_block_mask + static_cast<size_t>(p0 + p) * bm * bn;
        for (int idx = threadIdx.x; idx < chunks_per_tile; idx += blockDim.x) {
            const int r = idx / chunks_per_tile_row, cc = idx - r * chunks_per_tile_row;
            const size_t src = (static_cast<size_t>(brow) * bm + r) * seq_len + static_cast<size_t>(c) * bn + cc * 8;
            __half h[8];
            if (F32) {
                const float4 a = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(mask) + src));
                const float4 b = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(mask) + src + 4));
                h[0] = __float2half_rn(a.x); h[1] = __float2half_rn(a.y); h[2] = __float2half_rn(a.z); h[3] = __float2half_rn(a.w);
                h[4] = __float2half_rn(b.x); h[5] = __float2half_rn(b.y); h[6] = __float2half_rn(b.z); h[7] = __float2half_rn(b.w);
            } else {
                *reinterpret_cast<uint4*>(h) = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(mask) + src));
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = __hmul(neg, __hsub(one, h[i]));
            *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * bn + cc * 8) = *reinterpret_cast<uint4*>(h);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Scratch for stof_mask_compact_static: lives in the module's device image instead of a caller
// allocation.  Every GPU that loads the library holds these bytes until the process exits.
// ---------------------------------------------------------------------------------------------
constexpr int STATIC_MAX_TILES = 1 << 20;           // block rows x block columns the static scratch can classify
static __device__ __align__(256) unsigned char g_static_scratch[WS_HEADER + STATIC_MAX_TILES];

// Same ranking and gather as fill_kernel, but every write is checked against the capacity of the caller's
// buffers (the caller sized them without knowing the counts): entries that do not fit are dropped.
template <bool F32>
__global__ void __launch_bounds__(FILL_THREADS)
fill_bounded_kernel(const void* __restrict__ mask, int seq_len, int bm, int bn, const unsigned char* __restrict__ cls,
                    const int* __restrict__ full_row_ptr, const int* __restrict__ part_row_ptr, const int* __restrict__ load_row_ptr,
                    int* full_col_idx, int* part_col_idx, int* load_col_idx, long long col_capacity, __half* part_block_mask,
                    long long part_capacity) {
    extern __shared__ int s_part_cols[];
    const int nbn = seq_len / bn;
    const int brow = blockIdx.x, share = blockIdx.y, shares = gridDim.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int f0 = full_row_ptr[brow], p0 = part_row_ptr[brow], l0 = load_row_ptr[brow];
    const int n_part = part_row_ptr[brow + 1] - p0;
    if (warp == 0) {
        int nf = 0, np = 0;
        for (int c0 = 0; c0 < nbn; c0 += 32) {
            const int c = c0 + lane;
            const int k = c < nbn ? cls[static_cast<size_t>(brow) * nbn + c] : CLS_EMPTY;
            const unsigned bf = __ballot_sync(0xffffffffu, k == CLS_FULL);
            const unsigned bp = __ballot_sync(0xffffffffu, k == CLS_PART);
            const unsigned lt = (1u << lane) - 1u;
            const int rf = nf + __popc(bf & lt), rp = np + __popc(bp & lt);
            if (k == CLS_FULL) {
                if (share == 0) {
                    if (f0 + rf < col_capacity) full_col_idx[f0 + rf] = c;
                    if (l0 + rf + rp < col_capacity) load_col_idx[l0 + rf + rp] = c;
                }
            } else if (k == CLS_PART) {
                s_part_cols[rp] = c;
                if (share == 0) {
                    if (p0 + rp < col_capacity) part_col_idx[p0 + rp] = c;
                    if (l0 + rf + rp < col_capacity) load_col_idx[l0 + rf + rp] = c;
                }
            }
            nf += __popc(bf);
            np += __popc(bp);
        }
    }
    __syncthreads();
    if (n_part == 0 || part_block_mask == nullptr) return;
    const int chunks_per_tile_row = bn / 8;
    const int chunks_per_tile = bm * chunks_per_tile_row;
    const __half one = __float2half(1.0f), neg = __float2half(-10000.0f);
    for (int p = share; p < n_part; p += shares) {
        if (p0 + p >= part_capacity) break;
        const int c = s_part_cols[p];
        __half* dst = part_block_mask + static_cast<size_t>(p0 + p) * bm * bn;
        for (int idx = threadIdx.x; idx < chunks_per_tile; idx += blockDim.x) {
            const int r = idx / chunks_per_tile_row, cc = idx - r * chunks_per_tile_row;
            const size_t src = (static_cast<size_t>(brow) * bm + r) * seq_len + static_cast<size_t>(c) * bn + cc * 8;
            __half h[8];
            if (F32) {
                const float4 a = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(mask) + src));
                const float4 b = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(mask) + src + 4));
                h[0] = __float2half_rn(a.x); h[1] = __float2half_rn(a.y); h[2] = __float2half_rn(a.z); h[3] = __float2half_rn(a.w);
                h[4] = __float2half_rn(b.x); h[5] = __float2half_rn(b.y); h[6] = __float2half_rn(b.z); h[7] = __float2half_rn(b.w);
            } else {
                *reinterpret_cast<uint4*>(h) = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(mask) + src));
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = __hmul(neg, __hsub(one, h[i]));
            *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * bn + cc * 8) = *reinterpret_cast<uint4*>(h);
        }
    }
}

// Device address of g_static_scratch on the current device.  In host code the array's name is only a
// host-side handle, never a pointer a kernel may use, so the address is asked from the runtime once per
// device (with that device current) and cached.  The query may be what makes the runtime load the module (and
// with it the array) onto the device; the cached address dies with the device's primary context, so a
// cudaDeviceReset() on that device leaves it stale.
int static_scratch_address(unsigned char** out) {
    static std::mutex mu;
    static unsigned char* addr[64] = {};
    int dev = 0;
    STOF_CUDA(cudaGetDevice(&dev));
    STOF_REQUIRE(dev >= 0 && dev < 64, "mask_compact_static: device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        STOF_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        STOF_REQUIRE(p != nullptr, "mask_compact_static: the runtime returned no address for the scratch array");
        addr[dev] = static_cast<unsigned char*>(p);
    }
    *out = addr[dev];
    return STOF_OK;
}

int check_geometry(int seq_len, int bm, int bn) {
    STOF_REQUIRE(seq_len > 0 && bm > 0 && bn > 0, "mask compaction: seq_len/block sizes must be positive");
    STOF_REQUIRE(seq_len % bm == 0 && seq_len % bn == 0, "mask compaction: seq_len %d is not a multiple of block_m %d and block_n %d",
                 seq_len, bm, bn);
    STOF_REQUIRE(bn % 8 == 0, "mask compaction: block_n %d must be a multiple of 8", bn);
    STOF_REQUIRE(seq_len / bn <= MAX_TILES_PER_STRIPE, "mask compaction: more than %d tiles per row", MAX_TILES_PER_STRIPE);
    return STOF_OK;
}

}  // namespace
}  // namespace stof

using namespace stof;

extern "C" size_t stof_mask_workspace_bytes(int seq_len, int block_m, int block_n) {
    if (seq_len <= 0 || block_m <= 0 || block_n <= 0) return 0;
    return WS_HEADER + cls_bytes(seq_len / block_m, seq_len / block_n);
}

extern "C" int stof_mask_classify(const void* mask, int mask_dtype, int batch, int seq_len, int block_m, int block_n,
                                  int* full_row_ptr, int* part_row_ptr, int* load_row_ptr, long long* counts, void* workspace,
                                  size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (int rc = check_geometry(seq_len, block_m, block_n)) return rc;
    STOF_REQUIRE(mask && full_row_ptr && part_row_ptr && load_row_ptr && counts && workspace, "mask_classify: null pointer");
    STOF_REQUIRE(mask_dtype == STOF_DTYPE_F16 || mask_dtype == STOF_DTYPE_F32, "mask_classify: mask_dtype must be f16 or f32");
    STOF_REQUIRE(batch >= 1 && batch <= 65535, "mask_classify: batch %d out of range", batch);
    STOF_REQUIRE(aligned16(mask), "mask_classify: mask must be 16-byte aligned");
    if (workspace_bytes < stof_mask_workspace_bytes(seq_len, block_m, block_n)) {
        set_error("mask_classify: workspace of %zu bytes, need %zu", workspace_bytes, stof_mask_workspace_bytes(seq_len, block_m, block_n));
        return STOF_E_WORKSPACE;
    }
    const int nbm = seq_len / block_m;
    STOF_REQUIRE(nbm <= 65535, "mask_classify: more than 65535 block rows");
    // stripe width: whole tiles, at least 128 columns (256-byte row segments) for coalescing, enough stripes to fill the GPU
    int unit = block_n;
    while (unit < 128 && unit < seq_len) unit += block_n;
    const int units = (seq_len + unit - 1) / unit;
    int want = (4 * sm_count() + nbm * batch - 1) / (nbm * batch);
    if (want < 1) want = 1;
    if (want > units) want = units;
    const int units_per_stripe = (units + want - 1) / want;
    const int stripe_cols = units_per_stripe * unit;
    const int stripes = (seq_len + stripe_cols - 1) / stripe_cols;

    Workspace* ws = static_cast<Workspace*>(workspace);
    unsigned char* cls = static_cast<unsigned char*>(workspace) + WS_HEADER;
    STOF_CUDA(cudaMemsetAsync(ws, 0, WS_HEADER, stream));
    STOF_CUDA(cudaMemsetAsync(counts, 0, 4 * sizeof(long long), stream));
    dim3 grid(stripes, nbm, batch);
    if (mask_dtype == STOF_DTYPE_F32)
        classify_kernel<true><<<grid, CLASSIFY_THREADS, 0, stream>>>(mask, seq_len, block_m, block_n, stripe_cols, full_row_ptr, part_row_ptr,
                                                                      load_row_ptr, reinterpret_cast<unsigned long long*>(counts), ws, cls);
    else
        classify_kernel<false><<<grid, CLASSIFY_THREADS, 0, stream>>>(mask, seq_len, block_m, block_n, stripe_cols, full_row_ptr, part_row_ptr,
                                                                       load_row_ptr, reinterpret_cast<unsigned long long*>(counts), ws, cls);
    STOF_CUDA(cudaGetLastError());
    return STOF_OK;
}

extern "C" int stof_mask_fill(const void* mask, int mask_dtype, int seq_len, int block_m, int block_n, const int* full_row_ptr,
                              const int* part_row_ptr, const int* load_row_ptr, int* full_col_idx, int* part_col_idx,
                              int* load_col_idx, void* part_block_mask, const void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (int rc = check_geometry(seq_len, block_m, block_n)) return rc;
    STOF_REQUIRE(mask && full_row_ptr && part_row_ptr && load_row_ptr && workspace, "mask_fill: null pointer");
    STOF_REQUIRE(mask_dtype == STOF_DTYPE_F16 || mask_dtype == STOF_DTYPE_F32, "mask_fill: mask_dtype must be f16 or f32");
    STOF_REQUIRE(aligned16(mask) && (part_block_mask == nullptr || aligned16(part_block_mask)), "mask_fill: 16-byte alignment required");
    if (workspace_bytes < stof_mask_workspace_bytes(seq_len, block_m, block_n)) {
        set_error("mask_fill: workspace of %zu bytes, need %zu", workspace_bytes, stof_mask_workspace_bytes(seq_len, block_m, block_n));
        return STOF_E_WORKSPACE;
    }
    const int nbm = seq_len / block_m, nbn = seq_len / block_n;
    const unsigned char* cls = static_cast<const unsigned char*>(workspace) + WS_HEADER;
    int shares = (4 * sm_count() + nbm - 1) / nbm;
    if (shares < 1) shares = 1;
    if (shares > 8) shares = 8;
    if (part_block_mask == nullptr) shares = 1;
    dim3 grid(nbm, shares);
    const size_t smem = static_cast<size_t>(nbn) * sizeof(int);
    if (mask_dtype == STOF_DTYPE_F32)
        fill_kernel<true><<<grid, FILL_THREADS, smem, stream>>>(mask, seq_len, block_m, block_n, cls, full_row_ptr, part_row_ptr, load_row_ptr,
                                                                full_col_idx, part_col_idx, load_col_idx, static_cast<__half*>(part_block_mask));
    else
        fill_kernel<false><<<grid, FILL_THREADS, smem, stream>>>(mask, seq_len, block_m, block_n, cls, full_row_ptr, part_row_ptr, load_row_ptr,
                                                                 full_col_idx, part_col_idx, load_col_idx, static_cast<__half*>(part_block_mask));
    STOF_CUDA(cudaGetLastError());
    return STOF_OK;
}

// One call, nothing allocated: classify + fill with the scratch in the library's own device image (see the header).
extern "C" int stof_mask_compact_static(const void* mask, int mask_dtype, int batch, int seq_len, int block_m, int block_n,
                                        int* full_row_ptr, int* part_row_ptr, int* load_row_ptr, int* full_col_idx, int* part_col_idx,
                                        int* load_col_idx, long long col_capacity, void* part_block_mask, long long part_capacity,
                                        long long* counts, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (int rc = check_geometry(seq_len, block_m, block_n)) return rc;
    STOF_REQUIRE(mask && full_row_ptr && part_row_ptr && load_row_ptr && full_col_idx && part_col_idx && load_col_idx && counts,
                 "mask_compact_static: null pointer");
    STOF_REQUIRE(mask_dtype == STOF_DTYPE_F16 || mask_dtype == STOF_DTYPE_F32, "mask_compact_static: mask_dtype must be f16 or f32");
    STOF_REQUIRE(batch >= 1 && batch <= 65535, "mask_compact_static: batch %d out of range", batch);
    STOF_REQUIRE(col_capacity >= 0 && part_capacity >= 0, "mask_compact_static: negative capacity");
    STOF_REQUIRE(aligned16(mask) && (part_block_mask == nullptr || aligned16(part_block_mask)), "mask_compact_static: 16-byte alignment required");
    const int nbm = seq_len / block_m, nbn = seq_len / block_n;
    STOF_REQUIRE(nbm <= 65535, "mask_compact_static: more than 65535 block rows");
    if (static_cast<long long>(nbm) * nbn > STATIC_MAX_TILES) {
        set_error("mask_compact_static: %d x %d blocks exceed the %d tiles the built-in scratch holds; use stof_mask_classify / stof_mask_fill "
                  "with a workspace of your own", nbm, nbn, STATIC_MAX_TILES);
        return STOF_E_LIMIT;
    }
    unsigned char* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    Workspace* ws = reinterpret_cast<Workspace*>(scratch);
    unsigned char* cls = scratch + WS_HEADER;

    int unit = block_n;
    while (unit < 128 && unit < seq_len) unit += block_n;
    const int units = (seq_len + unit - 1) / unit;
    int want = (4 * sm_count() + nbm * batch - 1) / (nbm * batch);
    if (want < 1) want = 1;
    if (want > units) want = units;
    const int units_per_stripe = (units + want - 1) / want;
    const int stripe_cols = units_per_stripe * unit;
    const int stripes = (seq_len + stripe_cols - 1) / stripe_cols;

    // the array keeps what the previous call left: the ticket and the totals must start at zero
    STOF_CUDA(cudaMemsetAsync(ws, 0, WS_HEADER, stream));
    STOF_CUDA(cudaMemsetAsync(counts, 0, 4 * sizeof(long long), stream));
    dim3 grid(stripes, nbm, batch);
    if (mask_dtype == STOF_DTYPE_F32)
        classify_kernel<true><<<grid, CLASSIFY_THREADS, 0, stream>>>(mask, seq_len, block_m, block_n, stripe_cols, full_row_ptr, part_row_ptr,
                                                                      load_row_ptr, reinterpret_cast<unsigned long long*>(counts), ws, cls);
    else
        classify_kernel<false><<<grid, CLASSIFY_THREADS, 0, stream>>>(mask, seq_len, block_m, block_n, stripe_cols, full_row_ptr, part_row_ptr,
                                                                       load_row_ptr, reinterpret_cast<unsigned long long*>(counts), ws, cls);
    STOF_CUDA(cudaGetLastError());
    int shares = (4 * sm_count() + nbm - 1) / nbm;
    if (shares < 1) shares = 1;
    if (shares > 8) shares = 8;
    if (part_block_mask == nullptr) shares = 1;
    const size_t smem = static_cast<size_t>(nbn) * sizeof(int);
    dim3 fgrid(nbm, shares);
    if (mask_dtype == STOF_DTYPE_F32)
        fill_bounded_kernel<true><<<fgrid, FILL_THREADS, smem, stream>>>(mask, seq_len, block_m, block_n, cls, full_row_ptr, part_row_ptr, load_row_ptr,
                                                                         full_col_idx, part_col_idx, load_col_idx, col_capacity,
                                                                         static_cast<__half*>(part_block_mask), part_capacity);
    else
        fill_bounded_kernel<false><<<fgrid, FILL_THREADS, smem, stream>>>(mask, seq_len, block_m, block_n, cls, full_row_ptr, part_row_ptr, load_row_ptr,
                                                                          full_col_idx, part_col_idx, load_col_idx, col_capacity,
                                                                          static_cast<__half*>(part_block_mask), part_capacity);
    STOF_CUDA(cudaGetLastError());
    return STOF_OK;
}
