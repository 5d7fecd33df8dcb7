// C[M,N] = epilogue(A[M,K] @ W[K,N] + bias) with PAIRS of thread blocks on one 256 x 256 output tile (tcgen05 cta_group::2).
//
// Two thread blocks on neighbouring SMs (a cluster of 2) share each tile: block r of the pair owns rows r*128 .. r*128+127
// of the tile (its accumulator is 128 lanes x 256 fp32 columns of its own tensor memory) and stages, per K step of 64, its
// own 128 rows of A and 128 of the 256 columns of W; one tcgen05.mma.cta_group::2 issued by the leader (block 0) multiplies
// the pair's A halves with both W halves.  Per SM and per flop that is half the W bytes through shared memory, TMA and L2 of
// the one-block kernel, which is what the power-capped rate of long GEMMs depends on.
//   warp 8      TMA producer (both blocks): own A box and two 64 x 64 W boxes per stage, 6 stages of 32 KB; every copy
//               reports its bytes to the LEADER's full barrier (the leader arms it for both blocks' bytes)
//   warp 9      leader only: MMA issuer, two 256-column accumulators; after the MMAs of a stage (a tile) it commits twice,
//               once on its own "stage free" ("accumulator full") barrier and once on its peer's, by mapped address
//   warps 0-7   epilogue (both blocks), same as the one-block kernel; the peer's warps report "accumulator drained" to the
//               leader's barrier with remote mbarrier arrives
// Every copy and every commit names exactly one block's barrier.  Both blocks meet at a cluster barrier before they leave, so
// that neither frees shared or tensor memory its peer may still signal, read or write.
#include <atomic>
#include "stof_host.h"
#include "stof_ptx.cuh"
#include "stof_epilogue.cuh"

namespace stof {
namespace {

constexpr int P_BM = 128, P_BN = 256, P_BK = 64;          // per block: 128 rows x 256 columns of the pair's 256 x 256 tile
constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = P_BM * P_BK * 2;                 // 16 KB
constexpr int P_B_BYTES = P_BK * (P_BN / 2) * 2;           // 16 KB: this block's 128 of the 256 W columns
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_EPI_WARPS = 8;
constexpr int P_THREADS = (P_EPI_WARPS + 2) * 32;
constexpr int P_TMEM_COLS = 512;
constexpr int P_SLAB_BYTES = 32 * 64 * 2;
constexpr size_t P_SMEM = 1024 + static_cast<size_t>(P_STAGES) * P_STAGE_BYTES + P_EPI_WARPS * P_SLAB_BYTES + 256;

enum { PB_FULL = 0, PB_EMPTY = P_STAGES, PB_TFULL = 2 * P_STAGES, PB_TEMPTY = 2 * P_STAGES + 2, PB_COUNT = 2 * P_STAGES + 4 };

__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void mma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on the mbarrier at this cluster address (the leader's own or its peer's) once every MMA issued so far has completed
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_c,
                 const __half* __restrict__ bias, const __half* __restrict__ residual, long long ldr, int m, int n, int k, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* slabs = smem + P_STAGES * P_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(slabs + P_EPI_WARPS * P_SLAB_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + PB_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int tiles_n = (n + P_BN - 1) / P_BN, tiles_m = (m + 2 * P_BM - 1) / (2 * P_BM);
    const int num_tiles = tiles_m * tiles_n;
    const int kblocks = (k + P_BK - 1) / P_BK;
    const WaitCtx wctx{abort_flag, status};

    if (threadIdx.x == 0) {
        *abort_flag = (status != nullptr && *status != 0) ? 1 : 0;
        for (int i = 0; i < P_STAGES; ++i) {
            mbar_init(&bars[PB_FULL + i], 1);                 // the leader's: its own arrive.expect_tx; bytes from both blocks
            mbar_init(&bars[PB_EMPTY + i], 1);                // a tcgen05.commit of the leader, in both blocks
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars[PB_TFULL + i], 1);                // a tcgen05.commit of the leader, in both blocks
            mbar_init(&bars[PB_TEMPTY + i], 2 * P_EPI_WARPS); // the leader's: the epilogue warps of both blocks
        }
        fence_mbar_init();
    }
    if (warp == P_EPI_WARPS + 1) {
        tmem_alloc_pair(tmem_slot, P_TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                       // both blocks' barriers exist before any remote arrive or copy
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (*abort_flag == 0) {
        if (warp == P_EPI_WARPS) {
            // ------------------------------------------------------------------ TMA producer (both blocks)
            if (elect_one()) {
                tma_prefetch_desc(&map_a);
                tma_prefetch_desc(&map_w);
                int it = 0;
                for (int t = pair; t < num_tiles; t += pairs) {
                    const int m0 = (t / tiles_n) * (2 * P_BM) + static_cast<int>(rank) * P_BM;
                    const int n0 = (t % tiles_n) * P_BN + static_cast<int>(rank) * (P_BN / 2);
                    for (int kb = 0; kb < kblocks; ++kb, ++it) {
                        const int s = it % P_STAGES;
                        const uint32_t ph = (it / P_STAGES) & 1;
                        mbar_wait(&bars[PB_EMPTY + s], ph ^ 1, wctx, PB_EMPTY + s);
                        if (leader) mbar_arrive_expect_tx(&bars[PB_FULL + s], 2 * P_STAGE_BYTES);
                        const uint32_t full = map_to_rank(smem_u32(&bars[PB_FULL + s]), 0);
                        unsigned char* a_dst = smem + s * P_STAGE_BYTES;
                        unsigned char* b_dst = a_dst + P_A_BYTES;
                        tma_load_2d_pair(a_dst, &map_a, full, kb * P_BK, m0);
#pragma unroll
                        for (int j = 0; j < P_BN / 128; ++j)
                            tma_load_2d_pair(b_dst + j * (P_BK * 64 * 2), &map_w, full, n0 + 64 * j, kb * P_BK);
                    }
                }
            }
        } else if (warp == P_EPI_WARPS + 1) {
            // ------------------------------------------------------------------ MMA issuer (leader only)
            if (leader && elect_one()) {
                constexpr uint32_t idesc = make_idesc_f16(2 * P_BM, P_BN, /*b_mn_major=*/true);
                int it = 0, local = 0;
                for (int t = pair; t < num_tiles; t += pairs, ++local) {
                    const int acc = local & 1;
                    const uint32_t acc_ph = (local >> 1) & 1;
                    mbar_wait(&bars[PB_TEMPTY + acc], acc_ph ^ 1, wctx, PB_TEMPTY + acc);
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc * P_BN;
                    for (int kb = 0; kb < kblocks; ++kb, ++it) {
                        const int s = it % P_STAGES;
                        const uint32_t ph = (it / P_STAGES) & 1;
                        mbar_wait(&bars[PB_FULL + s], ph, wctx, PB_FULL + s);
                        tc_fence_after();
                        const uint32_t a_addr = smem_u32(smem + s * P_STAGE_BYTES);
                        const uint32_t b_addr = a_addr + P_A_BYTES;
#pragma unroll
                        for (int kk = 0; kk < P_BK / 16; ++kk) {
                            const uint64_t a_desc = make_smem_desc_sw128(a_addr + kk * 32, 16, 1024);
                            const uint64_t b_desc = make_smem_desc_sw128(b_addr + kk * 2048, P_BK * 64 * 2, 1024);
                            mma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                        }
                        // the stage is free in both blocks: one commit per block's barrier
                        tc_commit_pair(smem_u32(&bars[PB_EMPTY + s]));
                        tc_commit_pair(map_to_rank(smem_u32(&bars[PB_EMPTY + s]), 1));
                    }
                    tc_commit_pair(smem_u32(&bars[PB_TFULL + acc]));
                    tc_commit_pair(map_to_rank(smem_u32(&bars[PB_TFULL + acc]), 1));
                }
            }
        } else {
            // ------------------------------------------------------------------ epilogue (both blocks)
            const int quarter = warp & 3, half_n = warp >> 2;
            unsigned char* slab = slabs + warp * P_SLAB_BYTES;
            int local = 0;
            for (int t = pair; t < num_tiles; t += pairs, ++local) {
                const int acc = local & 1;
                const uint32_t acc_ph = (local >> 1) & 1;
                const int m0 = (t / tiles_n) * (2 * P_BM) + static_cast<int>(rank) * P_BM, n0 = (t % tiles_n) * P_BN;
                const int row0 = m0 + quarter * 32;
                const int row = row0 + lane;
                const int colbase = n0 + half_n * (P_BN / 2);
                uint4 res[2][8];
                if (EPI == STOF_EPI_BIAS_RESIDUAL) {
#pragma unroll
                    for (int ch = 0; ch < 2; ++ch)
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            const int col = colbase + ch * 64 + g * 8;
                            res[ch][g] = (row < m && col < n) ? __ldg(reinterpret_cast<const uint4*>(residual + static_cast<size_t>(row) * ldr + col))
                                                              : make_uint4(0u, 0u, 0u, 0u);
                        }
                }
                mbar_wait(&bars[PB_TFULL + acc], acc_ph, wctx, PB_TFULL + acc);
                tc_fence_after();
                const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * P_BN + half_n * (P_BN / 2);
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t r0[32], r1[32];
                    tmem_ld32(t_row + ch * 64, r0);
                    tmem_ld32(t_row + ch * 64 + 32, r1);
                    tc_wait_ld();
                    if (ch == 1) {
                        // both chunks of this accumulator half are in registers: hand the accumulator back to the leader's MMA warp
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (leader) mbar_arrive(&bars[PB_TEMPTY + acc]);
                            else remote_arrive(map_to_rank(smem_u32(&bars[PB_TEMPTY + acc]), 0));
                        }
                    }
                    const int col0 = colbase + ch * 64;
                    if (col0 < n && row0 < m) {
                        if (lane == 0) tma_store_wait_read();
                        __syncwarp();
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            const uint32_t* src = (g < 4) ? &r0[8 * g] : &r1[8 * (g - 4)];
                            const int col = col0 + 8 * g;
                            float2 v[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) v[j] = pk2(__uint_as_float(src[2 * j]), __uint_as_float(src[2 * j + 1]));
                            if (bias != nullptr && col < n) {
                                const uint4 bu = __ldg(reinterpret_cast<const uint4*>(bias + col));
                                const __half2* bh = reinterpret_cast<const __half2*>(&bu);
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float2 f = __half22float2(bh[j]);
                                    v[j] = add2(v[j], pk2(f.x, f.y));
                                }
                            }
                            if (EPI == STOF_EPI_BIAS_GELU_ERF) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) v[j] = gelu_erf2(v[j]);
                            } else if (EPI == STOF_EPI_BIAS_GELU_TANH) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) v[j] = gelu_tanh2(v[j]);
                            } else if (EPI == STOF_EPI_BIAS_RELU) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    float x0, x1;
                                    upk2(v[j], x0, x1);
                                    v[j] = pk2(fmaxf(x0, 0.0f), fmaxf(x1, 0.0f));
                                }
                            } else if (EPI == STOF_EPI_BIAS_RESIDUAL) {
                                const __half2* rh = reinterpret_cast<const __half2*>(&res[ch][g]);
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float2 f = __half22float2(rh[j]);
                                    v[j] = add2(v[j], pk2(f.x, f.y));
                                }
                            }
                            uint4 o;
                            float lo, hi;
                            upk2(v[0], lo, hi); o.x = pack_half2(lo, hi);
                            upk2(v[1], lo, hi); o.y = pack_half2(lo, hi);
                            upk2(v[2], lo, hi); o.z = pack_half2(lo, hi);
                            upk2(v[3], lo, hi); o.w = pack_half2(lo, hi);
                            *reinterpret_cast<uint4*>(slab + lane * 128 + ((g ^ (lane & 7)) << 4)) = o;
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d(&map_c, slab, col0, row0);
                            tma_store_commit();
                        }
                    }
                }
            }
            if (lane == 0) tma_store_wait_all();
        }
    }
    // neither block leaves while its peer may still signal one of its barriers, read its shared memory or write its tensor memory
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == P_EPI_WARPS + 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, P_TMEM_COLS);
    }
}

template <int EPI>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mc, const __half* bias, const __half* residual, long long ldr,
                int m, int n, int k, int* status, cudaStream_t stream) {
    static std::atomic<bool> configured[64];     // per device; host threads may race here, every one of them stores the same value
    int dev = 0;
    STOF_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        STOF_CUDA(cudaFuncSetAttribute(gemm_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(P_SMEM)));
        configured[dev] = true;
    }
    const int tiles = ((m + 2 * P_BM - 1) / (2 * P_BM)) * ((n + P_BN - 1) / P_BN);
    int pairs = sm_count() / 2;
    if (pairs > tiles) pairs = tiles;
    gemm_pair_kernel<EPI><<<2 * pairs, P_THREADS, P_SMEM, stream>>>(ma, mw, mc, bias, residual, ldr, m, n, k, status);
    STOF_CUDA(cudaGetLastError());
    return STOF_OK;
}

}  // namespace

// Called by stof_gemm_bias_act for shapes with enough 256 x 256 tiles; the tensor maps are the one-block kernel's
// (A boxes of 128 rows x 64, W boxes of 64 x 64, C boxes of 32 rows x 64 columns).
int gemm_pair_dispatch(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mc, const __half* bias, const __half* residual,
                       long long ldr, int m, int n, int k, int epilogue, int* status, cudaStream_t stream) {
    switch (epilogue) {
        case STOF_EPI_BIAS: return launch_pair<STOF_EPI_BIAS>(ma, mw, mc, bias, residual, ldr, m, n, k, status, stream);
        case STOF_EPI_BIAS_GELU_ERF: return launch_pair<STOF_EPI_BIAS_GELU_ERF>(ma, mw, mc, bias, residual, ldr, m, n, k, status, stream);
        case STOF_EPI_BIAS_GELU_TANH: return launch_pair<STOF_EPI_BIAS_GELU_TANH>(ma, mw, mc, bias, residual, ldr, m, n, k, status, stream);
        case STOF_EPI_BIAS_RELU: return launch_pair<STOF_EPI_BIAS_RELU>(ma, mw, mc, bias, residual, ldr, m, n, k, status, stream);
        default: return launch_pair<STOF_EPI_BIAS_RESIDUAL>(ma, mw, mc, bias, residual, ldr, m, n, k, status, stream);
    }
}

}  // namespace stof
