// Block-masked multi-head attention for sm_100a: TMA-fed tcgen05 MMAs with the accumulators in tensor
// memory, online softmax in registers, only listed K/V blocks ever loaded.
//
// One thread block owns 128 query rows of one (batch, head) and walks the union of the 64-wide K/V
// tiles that any of its row blocks lists (block sizes 16..128 are mapped onto this 128 x 64 tiling
// through a small per-block code table in shared memory: 0 absent, 1 full, 2+i partial tile i).
//   warp 4      TMA producer: Q tile once, then (K, V) tile pairs through a ring of stages
//   warp 5      MMA issuer:   S = Q K^T (128 x 64 x 64) into one of two S buffers in tensor memory, and
//               O += P V (128 x 64 x 64) with P read from tensor memory (fp16) and V consumed in its natural
//               (key-row major) layout through an MN-major descriptor
//   warps 0-3   softmax: one query row per thread (tensor-memory lane), scores via tcgen05.ld, masking per
//               row block, exp2 with the scale folded in, running max with lazy rescale of O (only when
//               the maximum grew by more than 2^8), P written back with tcgen05.st
// Row blocks that do not list a tile skip its exponentials (P = 0); tiles nobody lists are never loaded.
#include "stof_host.h"
#include "stof_ptx.cuh"

namespace stof {
namespace {

constexpr int A_TQ = 128, A_TKV = 64, A_D = 64;
constexpr int A_STAGES = 5;
constexpr int A_Q_BYTES = A_TQ * A_D * 2;         // 16 KB
constexpr int A_KV_BYTES = A_TKV * A_D * 2;       // 8 KB each for K and V
constexpr int A_STAGE_BYTES = 2 * A_KV_BYTES;
constexpr int A_THREADS = 192;
constexpr int A_TMEM_COLS = 256;
constexpr int A_COL_S = 0, A_COL_O = 128, A_COL_P = 192;   // S0 @0, S1 @64, O @128, P0 @192, P1 @224
constexpr int A_MAX_TABLE_BYTES = 24 * 1024;
constexpr float A_RESCALE_THRESHOLD = 8.0f;       // log2 units

enum {
    AB_Q = 0, AB_KV_FULL = 1, AB_KV_EMPTY = AB_KV_FULL + A_STAGES, AB_S_FULL = AB_KV_EMPTY + A_STAGES, AB_P_FULL = AB_S_FULL + 2,
    AB_PV_DONE = AB_P_FULL + 2, AB_COUNT = AB_PV_DONE + 2
};

struct AttnParams {
    __half* out;
    long long o_stride_b, o_stride_h, o_stride_s;
    const int* full_row_ptr;
    const int* full_col_idx;
    const int* part_row_ptr;
    const int* part_col_idx;
    const __half* part_block_mask;
    int batch, heads, seq_len;
    int bm, bn;
    int slot_s[3], slot_h[3], slot_b[3];   // coordinate slot (1..3) of row / head / batch in the q, k, v tensor maps
    float scale_log2;
    int* status;
};

__device__ __forceinline__ void tma_tile(void* dst, const CUtensorMap* map, uint64_t* bar, int row, int h, int b, int ss, int sh, int sb) {
    int c[4] = {0, 0, 0, 0};
    c[ss] = row;
    c[sh] = h;
    c[sb] = b;
    tma_load_4d(dst, map, bar, c[0], c[1], c[2], c[3]);
}

__global__ void __launch_bounds__(A_THREADS, 2)
block_attn_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* q_smem = smem;
    unsigned char* kv_smem = q_smem + A_Q_BYTES;
    unsigned char* tail = kv_smem + A_STAGES * A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + AB_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* n_tiles_smem = reinterpret_cast<int*>(tmem_slot + 2);
    uint16_t* tile_list = reinterpret_cast<uint16_t*>(tmem_slot + 4);
    const int n_kv_tiles_all = (p.seq_len + A_TKV - 1) / A_TKV;
    uint16_t* table = tile_list + ((n_kv_tiles_all + 7) & ~7);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
    const int nbm = p.seq_len / p.bm, ncb = p.seq_len / p.bn;
    const int nrb = A_TQ / p.bm;                       // row blocks per thread block (1..8)
    const WaitCtx wctx{abort_flag, p.status};

    // ------------------------------------------------------------------ prologue
    if (threadIdx.x == 0) {
        *abort_flag = (p.status != nullptr && *p.status != 0) ? 1 : 0;
        mbar_init(&bars[AB_Q], 1);
        for (int i = 0; i < A_STAGES; ++i) {
            mbar_init(&bars[AB_KV_FULL + i], 1);
            mbar_init(&bars[AB_KV_EMPTY + i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars[AB_S_FULL + i], 1);
            mbar_init(&bars[AB_P_FULL + i], 4);
            mbar_init(&bars[AB_PV_DONE + i], 1);
        }
        fence_mbar_init();
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, A_TMEM_COLS);
        tmem_relinquish();
    }
    for (int i = threadIdx.x; i < nrb * ncb; i += blockDim.x) table[i] = 0;
    __syncthreads();
    for (int lrb = 0; lrb < nrb; ++lrb) {
        const int rb = qt * nrb + lrb;
        if (rb >= nbm) break;
        const int f0 = p.full_row_ptr[rb], f1 = p.full_row_ptr[rb + 1];
        for (int i = f0 + threadIdx.x; i < f1; i += blockDim.x) {
            const int c = p.full_col_idx[i];
            if (c >= 0 && c < ncb) table[lrb * ncb + c] = 1;
            else if (p.status) atomicCAS(p.status, 0, STATUS_BAD_INDEX);
        }
        const int p0 = p.part_row_ptr[rb], p1 = p.part_row_ptr[rb + 1];
        for (int i = p0 + threadIdx.x; i < p1; i += blockDim.x) {
            const int c = p.part_col_idx[i];
            if (c >= 0 && c < ncb) table[lrb * ncb + c] = static_cast<uint16_t>(2 + (i - p0));
            else if (p.status) atomicCAS(p.status, 0, STATUS_BAD_INDEX);
        }
    }
    __syncthreads();
    if (warp == 0) {
        // ordered list of the 64-wide K/V tiles that at least one row block of this thread block lists
        int count = 0;
        for (int t0 = 0; t0 < n_kv_tiles_all; t0 += 32) {
            const int t = t0 + lane;
            bool active = false;
            if (t < n_kv_tiles_all) {
                const int c_lo = (t * A_TKV) / p.bn;
                const int c_hi = min(ncb - 1, (t * A_TKV + A_TKV - 1) / p.bn);
                for (int lrb = 0; lrb < nrb; ++lrb)
                    for (int c = c_lo; c <= c_hi; ++c) active |= table[lrb * ncb + c] != 0;
            }
            const unsigned bal = __ballot_sync(0xffffffffu, active);
            if (active) tile_list[count + __popc(bal & ((1u << lane) - 1u))] = static_cast<uint16_t>(t);
            count += __popc(bal);
        }
        if (lane == 0) *n_tiles_smem = count;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int n_tiles = *n_tiles_smem;
    const int q_row0 = qt * A_TQ;

    if (*abort_flag == 0 && n_tiles > 0) {
        if (warp == 4) {
            // -------------------------------------------------------------- TMA producer
            if (elect_one()) {
                tma_prefetch_desc(&map_q);
                tma_prefetch_desc(&map_k);
                tma_prefetch_desc(&map_v);
                mbar_arrive_expect_tx(&bars[AB_Q], A_Q_BYTES);
                tma_tile(q_smem, &map_q, &bars[AB_Q], q_row0, head, batch, p.slot_s[0], p.slot_h[0], p.slot_b[0]);
                for (int j = 0; j < n_tiles; ++j) {
                    const int s = j % A_STAGES;
                    const uint32_t ph = (j / A_STAGES) & 1;
                    mbar_wait(&bars[AB_KV_EMPTY + s], ph ^ 1, wctx, AB_KV_EMPTY + s);
                    const int kv_row = static_cast<int>(tile_list[j]) * A_TKV;
                    unsigned char* k_dst = kv_smem + s * A_STAGE_BYTES;
                    mbar_arrive_expect_tx(&bars[AB_KV_FULL + s], A_STAGE_BYTES);
                    tma_tile(k_dst, &map_k, &bars[AB_KV_FULL + s], kv_row, head, batch, p.slot_s[1], p.slot_h[1], p.slot_b[1]);
                    tma_tile(k_dst + A_KV_BYTES, &map_v, &bars[AB_KV_FULL + s], kv_row, head, batch, p.slot_s[2], p.slot_h[2], p.slot_b[2]);
                }
            }
        } else if (warp == 5) {
            // -------------------------------------------------------------- MMA issuer
            if (elect_one()) {
                constexpr uint32_t idesc_qk = make_idesc_f16(A_TQ, A_TKV, /*b_mn_major=*/false);
                constexpr uint32_t idesc_pv = make_idesc_f16(A_TQ, A_D, /*b_mn_major=*/true);
                const uint32_t q_addr = smem_u32(q_smem);
                mbar_wait(&bars[AB_Q], 0, wctx, AB_Q);
                auto issue_qk = [&](int j) {
                    const int s = j % A_STAGES;
                    mbar_wait(&bars[AB_KV_FULL + s], (j / A_STAGES) & 1, wctx, AB_KV_FULL + s);
                    tc_fence_after();
                    const uint32_t k_addr = smem_u32(kv_smem + s * A_STAGE_BYTES);
                    const uint32_t d = tmem_base + A_COL_S + (j & 1) * A_TKV;
#pragma unroll
                    for (int kk = 0; kk < A_D / 16; ++kk)
                        mma_f16_ss(d, make_smem_desc_sw128(q_addr + kk * 32, 16, 1024), make_smem_desc_sw128(k_addr + kk * 32, 16, 1024),
                                   idesc_qk, kk > 0 ? 1u : 0u);
                    tc_commit(&bars[AB_S_FULL + (j & 1)]);
                };
                issue_qk(0);
                for (int j = 0; j < n_tiles; ++j) {
                    if (j + 1 < n_tiles) issue_qk(j + 1);
                    const int b = j & 1, s = j % A_STAGES;
                    mbar_wait(&bars[AB_P_FULL + b], (j >> 1) & 1, wctx, AB_P_FULL + b);
                    tc_fence_after();
                    const uint32_t v_addr = smem_u32(kv_smem + s * A_STAGE_BYTES + A_KV_BYTES);
                    const uint32_t d = tmem_base + A_COL_O;
#pragma unroll
                    for (int kk = 0; kk < A_TKV / 16; ++kk) {
                        const uint64_t v_desc = make_smem_desc_sw128(v_addr + kk * 2048, 16, 1024);
                        const uint32_t acc = (j > 0 || kk > 0) ? 1u : 0u;
                        mma_f16_ts(d, tmem_base + A_COL_P + b * (A_TKV / 2) + kk * 8, v_desc, idesc_pv, acc);
                    }
                    tc_commit(&bars[AB_KV_EMPTY + s]);
                    tc_commit(&bars[AB_PV_DONE + b]);
                }
            }
        } else {
            // -------------------------------------------------------------- softmax warps (one row per thread)
            const int lr = warp * 32 + lane;                 // local row = tensor-memory lane
            const int row = q_row0 + lr;
            const int lrb = lr / p.bm;
            const int rb = qt * nrb + lrb;
            const bool rb_valid = rb < nbm;
            const int row_in_block = lr % p.bm;
            const int part_base = rb_valid ? p.part_row_ptr[rb] : 0;
            const uint16_t* my_table = table + lrb * ncb;
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
            float m_ref = -INFINITY, l_sum = 0.f;

            for (int j = 0; j < n_tiles; ++j) {
                const int b = j & 1;
                const int tile = tile_list[j];
                mbar_wait(&bars[AB_S_FULL + b], (j >> 1) & 1, wctx, AB_S_FULL + b);
                tc_fence_after();
                uint32_t raw[2][32];
                tmem_ld32(t_lane + A_COL_S + b * A_TKV, raw[0]);
                tmem_ld32(t_lane + A_COL_S + b * A_TKV + 32, raw[1]);
                tc_wait_ld();

                // codes of the four 16-column groups of this tile for this thread's row block
                int code[4];
                bool all_full = true, all_absent = true;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int col = tile * A_TKV + g * 16;
                    code[g] = (rb_valid && col < p.seq_len) ? my_table[col / p.bn] : 0;
                    all_full &= code[g] == 1;
                    all_absent &= code[g] == 0;
                }
                const bool warp_skip = __all_sync(0xffffffffu, all_absent);
                uint32_t packed[32];
                if (warp_skip) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) packed[i] = 0u;
                } else {
                    float s[64];
#pragma unroll
                    for (int i = 0; i < 64; ++i) s[i] = __uint_as_float(raw[i >> 5][i & 31]);
                    if (!__all_sync(0xffffffffu, all_full)) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if (code[g] == 0) {
#pragma unroll
                                for (int i = 0; i < 16; ++i) s[16 * g + i] = -INFINITY;
                            } else if (code[g] >= 2) {
                                const int col_in_block = (tile * A_TKV + g * 16) % p.bn;
                                const __half* mp = p.part_block_mask +
                                                   (static_cast<size_t>(part_base + code[g] - 2) * p.bm + row_in_block) * p.bn + col_in_block;
                                const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(mp));
                                const uint4 u1 = __ldg(reinterpret_cast<const uint4*>(mp + 8));
                                const __half2* h0 = reinterpret_cast<const __half2*>(&u0);
                                const __half2* h1 = reinterpret_cast<const __half2*>(&u1);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float2 a = __half22float2(h0[i]), c2 = __half22float2(h1[i]);
                                    s[16 * g + 2 * i] += a.x;
                                    s[16 * g + 2 * i + 1] += a.y;
                                    s[16 * g + 8 + 2 * i] += c2.x;
                                    s[16 * g + 8 + 2 * i + 1] += c2.y;
                                }
                            }
                        }
                    }
                    float mx = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        s[i] *= p.scale_log2;
                        mx = fmaxf(mx, s[i]);
                    }
                    // lazy rescale: move the reference maximum only when it would grow by more than the threshold
                    const bool need = mx > m_ref + A_RESCALE_THRESHOLD || (m_ref == -INFINITY && mx > -INFINITY);
                    if (__any_sync(0xffffffffu, need)) {
                        float alpha = 1.0f;
                        if (need) {
                            alpha = (m_ref == -INFINITY) ? 0.0f : fast_exp2(m_ref - mx);
                            m_ref = mx;
                            l_sum *= alpha;
                        }
                        if (j > 0) {
                            mbar_wait(&bars[AB_PV_DONE + ((j - 1) & 1)], ((j - 1) >> 1) & 1, wctx, AB_PV_DONE + ((j - 1) & 1));
                            tc_fence_after();
                            uint32_t o[2][32];
                            tmem_ld32(t_lane + A_COL_O, o[0]);
                            tmem_ld32(t_lane + A_COL_O + 32, o[1]);
                            tc_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                o[0][i] = __float_as_uint(__uint_as_float(o[0][i]) * alpha);
                                o[1][i] = __float_as_uint(__uint_as_float(o[1][i]) * alpha);
                            }
                            tmem_st32(t_lane + A_COL_O, o[0]);
                            tmem_st32(t_lane + A_COL_O + 32, o[1]);
                            tc_wait_st();
                        }
                    }
                    const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
                    float sum = 0.f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float e0 = fast_exp2(s[2 * i] - m_use), e1 = fast_exp2(s[2 * i + 1] - m_use);
                        sum += e0 + e1;
                        packed[i] = pack_half2(e0, e1);
                    }
                    l_sum += sum;
                }
                // P buffer b is free once the PV product of tile j-2 has completed
                if (j >= 2) mbar_wait(&bars[AB_PV_DONE + b], ((j - 2) >> 1) & 1, wctx, AB_PV_DONE + b);
                tc_fence_after();
                tmem_st32(t_lane + A_COL_P + b * (A_TKV / 2), packed);
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars[AB_P_FULL + b]);
            }
            // ---------------------------------------------------------- epilogue: O / l -> fp16 -> global
            const int last = n_tiles - 1;
            mbar_wait(&bars[AB_PV_DONE + (last & 1)], (last >> 1) & 1, wctx, AB_PV_DONE + (last & 1));
            tc_fence_after();
            uint32_t o[2][32];
            tmem_ld32(t_lane + A_COL_O, o[0]);
            tmem_ld32(t_lane + A_COL_O + 32, o[1]);
            tc_wait_ld();
            if (row < p.seq_len) {
                const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.0f;
                __half* dst = p.out + batch * p.o_stride_b + head * p.o_stride_h + static_cast<long long>(row) * p.o_stride_s;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint32_t* src = &o[c >> 2][(c & 3) * 8];
                    uint4 u;
                    u.x = pack_half2(__uint_as_float(src[0]) * inv, __uint_as_float(src[1]) * inv);
                    u.y = pack_half2(__uint_as_float(src[2]) * inv, __uint_as_float(src[3]) * inv);
                    u.z = pack_half2(__uint_as_float(src[4]) * inv, __uint_as_float(src[5]) * inv);
                    u.w = pack_half2(__uint_as_float(src[6]) * inv, __uint_as_float(src[7]) * inv);
                    *reinterpret_cast<uint4*>(dst + 8 * c) = u;
                }
            }
        }
    } else if (n_tiles == 0 && warp < 4) {
        // no listed key for any of these rows: the output is zero
        const int row = q_row0 + warp * 32 + lane;
        if (row < p.seq_len) {
            __half* dst = p.out + batch * p.o_stride_b + head * p.o_stride_h + static_cast<long long>(row) * p.o_stride_s;
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(dst + 8 * c) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, A_TMEM_COLS);
    }
}

size_t attn_smem_bytes(int seq_len, int bm, int bn) {
    const int n_kv_tiles_all = (seq_len + A_TKV - 1) / A_TKV;
    const size_t table = static_cast<size_t>(A_TQ / bm) * (seq_len / bn) * 2;
    return 1024 + A_Q_BYTES + static_cast<size_t>(A_STAGES) * A_STAGE_BYTES + AB_COUNT * 8 + 16 +
           static_cast<size_t>((n_kv_tiles_all + 7) & ~7) * 2 + table + 16;
}

// Sorts the three outer dimensions (row, head, batch) by stride so that the tensor map's strides ascend;
// returns the coordinate slot of each logical dimension.
int make_qkv_map(CUtensorMap* map, const void* base, int batch, int heads, int seq_len, const long long st[3], int box_rows, int slot_s[1],
                 int slot_h[1], int slot_b[1]) {
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

}  // namespace
}  // namespace stof

using namespace stof;

extern "C" int stof_block_attn(const void* q, const void* k, const void* v, void* out, int batch, int heads, int seq_len, int head_dim,
                               const long long q_strides[3], const long long k_strides[3], const long long v_strides[3],
                               const long long out_strides[3], const int* full_row_ptr, const int* full_col_idx, const int* part_row_ptr,
                               const int* part_col_idx, const void* part_block_mask, const int* load_row_ptr, const int* load_col_idx,
                               int block_m, int block_n, int num_warps, float softmax_scale, int* status_dev, void* stream_) {
    (void)load_row_ptr; (void)load_col_idx; (void)num_warps;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    STOF_REQUIRE(q && k && v && out, "block_attn: null q/k/v/out");
    STOF_REQUIRE(full_row_ptr && part_row_ptr, "block_attn: null row pointer array");
    STOF_REQUIRE(head_dim == A_D, "block_attn: head_dim %d unsupported (the kernels are built for 64, as the reference's are)", head_dim);
    STOF_REQUIRE(batch > 0 && heads > 0 && seq_len > 0, "block_attn: bad shape");
    STOF_REQUIRE(batch <= 65535 && heads <= 65535, "block_attn: batch/heads beyond 65535");
    STOF_REQUIRE(block_m == 16 || block_m == 32 || block_m == 64 || block_m == 128, "block_attn: BLOCK_M %d not in {16,32,64,128}", block_m);
    STOF_REQUIRE(block_n == 16 || block_n == 32 || block_n == 64 || block_n == 128, "block_attn: BLOCK_N %d not in {16,32,64,128}", block_n);
    STOF_REQUIRE(seq_len % block_m == 0 && seq_len % block_n == 0, "block_attn: seq_len %d not a multiple of BLOCK_M %d / BLOCK_N %d", seq_len,
                 block_m, block_n);
    STOF_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(part_block_mask),
                 "block_attn: pointers must be 16-byte aligned");
    const long long* all[4] = {q_strides, k_strides, v_strides, out_strides};
    for (int t = 0; t < 4; ++t) {
        STOF_REQUIRE(all[t] != nullptr, "block_attn: null stride array");
        for (int i = 0; i < 3; ++i)
            STOF_REQUIRE(all[t][i] > 0 && all[t][i] % 8 == 0, "block_attn: strides must be positive multiples of 8 elements");
    }
    const size_t table_bytes = static_cast<size_t>(A_TQ / block_m) * (seq_len / block_n) * 2;
    if (table_bytes > A_MAX_TABLE_BYTES) {
        set_error("block_attn: seq_len %d with %dx%d blocks needs a %zu-byte block table, beyond the maximum of %d", seq_len, block_m, block_n,
                  table_bytes, A_MAX_TABLE_BYTES);
        return STOF_E_LIMIT;
    }
    AttnParams p;
    p.out = static_cast<__half*>(out);
    p.o_stride_b = out_strides[0]; p.o_stride_h = out_strides[1]; p.o_stride_s = out_strides[2];
    p.full_row_ptr = full_row_ptr; p.full_col_idx = full_col_idx;
    p.part_row_ptr = part_row_ptr; p.part_col_idx = part_col_idx;
    p.part_block_mask = static_cast<const __half*>(part_block_mask);
    p.batch = batch; p.heads = heads; p.seq_len = seq_len; p.bm = block_m; p.bn = block_n;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.status = status_dev;
    CUtensorMap mq, mk, mv;
    if (int rc = make_qkv_map(&mq, q, batch, heads, seq_len, q_strides, A_TQ, &p.slot_s[0], &p.slot_h[0], &p.slot_b[0])) return rc;
    if (int rc = make_qkv_map(&mk, k, batch, heads, seq_len, k_strides, A_TKV, &p.slot_s[1], &p.slot_h[1], &p.slot_b[1])) return rc;
    if (int rc = make_qkv_map(&mv, v, batch, heads, seq_len, v_strides, A_TKV, &p.slot_s[2], &p.slot_h[2], &p.slot_b[2])) return rc;

    const size_t smem = attn_smem_bytes(seq_len, block_m, block_n);
    const dim3 grid((seq_len + A_TQ - 1) / A_TQ, heads, batch);
    static size_t configured_smem[64] = {};
    int dev = 0;
    STOF_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || configured_smem[dev] < smem) {
        STOF_CUDA(cudaFuncSetAttribute(block_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        if (dev >= 0 && dev < 64) configured_smem[dev] = smem;
    }
    block_attn_kernel<<<grid, A_THREADS, smem, stream>>>(mq, mk, mv, p);
    STOF_CUDA(cudaGetLastError());
    return STOF_OK;
}
