// Y[M,N] = LayerNorm(A[M,K] @ W[K,N] + bias + residual) * gamma + beta, with the row statistics taken inside the GEMM's
// epilogue (tcgen05 + TMEM + TMA), for N a multiple of 256 up to 1024.
//
// A LayerNorm row spans all N columns, a thread block's accumulator 256 of them, so the N / 256 thread blocks that hold the
// column slices of the same 128 rows form a CLUSTER along N and exchange per-row partial statistics through distributed shared
// memory.  Persistent: cluster c walks the 128-row blocks c, c + clusters, ...; block r of the cluster owns columns
// r * 256 .. r * 256 + 255 of every row block.
//   warp 8      TMA producer: A tile (128 rows x 64 k) and four 64 x 64 W boxes per stage, 3 stages of 48 KB (plain per-block
//               loads of this GPU's memory; every block of the cluster fetches the A tile itself, from L2 after the first)
//   warp 9      MMA issuer: 4 tcgen05.mma (128 x 256 x 16) per stage into one of two 256-column fp32 accumulators
//   warps 0-7   epilogue, one row (tensor-memory lane) and 128 columns per thread:
//               pass 1  x = accumulator + bias + residual (fp32), written back over the accumulator; the thread's mean and
//                       centred sum of squares over its 128 columns (two sweeps over registers, 32 columns at a time, merged
//                       by the parallel-variance formula) go into the partials table of EVERY block of the cluster (remote
//                       shared-memory stores), followed by one arrive per warp on that block's "partials complete" barrier
//               pass 2  once all 2 * N / 256 partials of a row have arrived, they are merged into the row's mean and 1 / sigma;
//                       x is read back from tensor memory, normalised, scaled by gamma, shifted by beta, packed to fp16 in a
//                       swizzled shared-memory slab and written with TMA stores
// The statistics are fp32 and taken before any rounding to fp16 (the unfused path rounds the GEMM output first).  The partials
// table and its barrier are double-buffered like the accumulators: a block may run at most one row block ahead of its peers,
// because it cannot complete row block t + 1 before every peer has contributed to it, which a peer's warp does only after it has
// finished reading the partials of row block t.
// All blocks of a cluster meet at a cluster barrier before they leave: nobody frees shared memory a peer may still write.
#include <cstdlib>
#include <atomic>
#include "stof_host.h"
#include "stof_ptx.cuh"

namespace stof {
namespace {

constexpr int L_BM = 128, L_BN = 256, L_BK = 64;
constexpr int L_STAGES = 3;
constexpr int L_A_BYTES = L_BM * L_BK * 2;            // 16 KB
constexpr int L_B_BYTES = L_BK * L_BN * 2;            // 32 KB
constexpr int L_STAGE_BYTES = L_A_BYTES + L_B_BYTES;  // 48 KB
constexpr int L_EPI_WARPS = 8;
constexpr int L_THREADS = (L_EPI_WARPS + 2) * 32;
constexpr int L_TMEM_COLS = 512;
constexpr int L_SLAB_BYTES = 32 * 64 * 2;
constexpr int L_MAX_CLUSTER = 4;                      // N <= 1024
// partials[accumulator][source block][column half][row] = {mean, centred sum of squares} of 128 columns
constexpr int L_PART_BYTES = 2 * L_MAX_CLUSTER * 2 * L_BM * 8;      // 16 KB
constexpr size_t L_SMEM = 1024 + static_cast<size_t>(L_STAGES) * L_STAGE_BYTES + L_EPI_WARPS * L_SLAB_BYTES + L_PART_BYTES + 256;

enum { LB_FULL = 0, LB_EMPTY = L_STAGES, LB_TFULL = 2 * L_STAGES, LB_TEMPTY = 2 * L_STAGES + 2, LB_PART = 2 * L_STAGES + 4,
       LB_COUNT = 2 * L_STAGES + 6 };

__device__ __forceinline__ void st_cluster_f32x2(uint32_t cluster_addr, float a, float b) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(cluster_addr), "f"(a), "f"(b) : "memory");
}

// merges (n_b, mean_b, m2_b) into (n_a, mean_a, m2_a): parallel variance (Chan et al.)
__device__ __forceinline__ void merge_stats(float& n_a, float& mean_a, float& m2_a, float n_b, float mean_b, float m2_b) {
    const float n = n_a + n_b;
    const float delta = mean_b - mean_a;
    const float f = n_b / n;
    mean_a = fmaf(delta, f, mean_a);
    m2_a = m2_a + m2_b + delta * delta * n_a * f;
    n_a = n;
}

__global__ void __launch_bounds__(L_THREADS, 1)
gemm_ln_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_c,
               const __half* __restrict__ bias, const __half* __restrict__ residual, long long ldr, const __half* __restrict__ gamma,
               const __half* __restrict__ beta, float eps, int m, int n, int k, int cluster_size, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* slabs = smem + L_STAGES * L_STAGE_BYTES;          // one 4 KB slab per epilogue warp, 1024-aligned
    float2* partials = reinterpret_cast<float2*>(slabs + L_EPI_WARPS * L_SLAB_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(partials) + L_PART_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + LB_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = static_cast<int>(cluster_rank());
    const int cluster_id = blockIdx.x / cluster_size, clusters = gridDim.x / cluster_size;
    const int tiles_m = (m + L_BM - 1) / L_BM;
    const int kblocks = (k + L_BK - 1) / L_BK;
    const int n0 = rank * L_BN;
    const WaitCtx wctx{abort_flag, status};

    if (threadIdx.x == 0) {
        *abort_flag = (status != nullptr && *status != 0) ? 1 : 0;
        for (int i = 0; i < L_STAGES; ++i) {
            mbar_init(&bars[LB_FULL + i], 1);
            mbar_init(&bars[LB_EMPTY + i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars[LB_TFULL + i], 1);
            mbar_init(&bars[LB_TEMPTY + i], L_EPI_WARPS);
            mbar_init(&bars[LB_PART + i], static_cast<uint32_t>(cluster_size * L_EPI_WARPS));          // every epilogue warp of the cluster
        }
        fence_mbar_init();
    }
    if (warp == L_EPI_WARPS + 1) {
        tmem_alloc(tmem_slot, L_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                       // every block's barriers exist before any remote store or arrive
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // The status word is read by every block on its own; a block that sat out while its peers ran would leave them waiting for
    // its partials until their wait budgets ran out.  So the decision to run is taken per cluster: every block tells every
    // peer through a flag in shared memory and all of them run only if none objects.
    __shared__ int peer_abort[L_MAX_CLUSTER];
    if (threadIdx.x < cluster_size) {
        const uint32_t dst = map_to_rank(smem_u32(&peer_abort[rank]), static_cast<uint32_t>(threadIdx.x));
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(dst), "r"(*abort_flag) : "memory");
    }
    cluster_sync_all();
    bool run = true;
    for (int i = 0; i < cluster_size; ++i) run = run && peer_abort[i] == 0;

    if (run) {
        if (warp == L_EPI_WARPS) {
            // ------------------------------------------------------------------ TMA producer
            if (elect_one()) {
                tma_prefetch_desc(&map_a);
                tma_prefetch_desc(&map_w);
                int it = 0;
                for (int rb = cluster_id; rb < tiles_m; rb += clusters) {
                    const int m0 = rb * L_BM;
                    for (int kb = 0; kb < kblocks; ++kb, ++it) {
                        const int s = it % L_STAGES;
                        const uint32_t ph = (it / L_STAGES) & 1;
                        mbar_wait(&bars[LB_EMPTY + s], ph ^ 1, wctx, LB_EMPTY + s);
                        unsigned char* a_dst = smem + s * L_STAGE_BYTES;
                        unsigned char* b_dst = a_dst + L_A_BYTES;
                        mbar_arrive_expect_tx(&bars[LB_FULL + s], L_STAGE_BYTES);
                        tma_load_2d(a_dst, &map_a, &bars[LB_FULL + s], kb * L_BK, m0);
#pragma unroll
                        for (int j = 0; j < L_BN / 64; ++j)
                            tma_load_2d(b_dst + j * (L_BK * 64 * 2), &map_w, &bars[LB_FULL + s], n0 + 64 * j, kb * L_BK);
                    }
                }
            }
        } else if (warp == L_EPI_WARPS + 1) {
            // ------------------------------------------------------------------ MMA issuer
            if (elect_one()) {
                constexpr uint32_t idesc = make_idesc_f16(L_BM, L_BN, /*b_mn_major=*/true);
                int it = 0, local = 0;
                for (int rb = cluster_id; rb < tiles_m; rb += clusters, ++local) {
                    const int acc = local & 1;
                    const uint32_t acc_ph = (local >> 1) & 1;
                    mbar_wait(&bars[LB_TEMPTY + acc], acc_ph ^ 1, wctx, LB_TEMPTY + acc);
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc * L_BN;
                    for (int kb = 0; kb < kblocks; ++kb, ++it) {
                        const int s = it % L_STAGES;
                        const uint32_t ph = (it / L_STAGES) & 1;
                        mbar_wait(&bars[LB_FULL + s], ph, wctx, LB_FULL + s);
                        tc_fence_after();
                        const uint32_t a_addr = smem_u32(smem + s * L_STAGE_BYTES);
                        const uint32_t b_addr = a_addr + L_A_BYTES;
#pragma unroll
                        for (int kk = 0; kk < L_BK / 16; ++kk) {
                            const uint64_t a_desc = make_smem_desc_sw128(a_addr + kk * 32, 16, 1024);
                            const uint64_t b_desc = make_smem_desc_sw128(b_addr + kk * 2048, L_BK * 64 * 2, 1024);
                            mma_f16_ss(d_tmem, a_desc, b_desc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                        }
                        tc_commit(&bars[LB_EMPTY + s]);
                    }
                    tc_commit(&bars[LB_TFULL + acc]);
                }
            }
        } else {
            // ------------------------------------------------------------------ epilogue
            const int quarter = warp & 3, half_n = warp >> 2;
            const int lrow = quarter * 32 + lane;                 // row inside the 128-row block = tensor-memory lane
            unsigned char* slab = slabs + warp * L_SLAB_BYTES;
            const float inv_n = 1.0f / static_cast<float>(n);
            int local = 0;
            for (int rb = cluster_id; rb < tiles_m; rb += clusters, ++local) {
                const int acc = local & 1;
                const uint32_t acc_ph = (local >> 1) & 1;
                const int row0 = rb * L_BM + quarter * 32;
                const int row = row0 + lane;
                const int colbase = n0 + half_n * (L_BN / 2);
                // the residual does not depend on the accumulator: its loads are in flight while the tile's MMAs finish
                uint4 res[2][8];
#pragma unroll
                for (int ch = 0; ch < 2; ++ch)
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        const int col = colbase + ch * 64 + g * 8;
                        res[ch][g] = (residual != nullptr && row < m) ? __ldg(reinterpret_cast<const uint4*>(residual + static_cast<size_t>(row) * ldr + col))
                                                                      : make_uint4(0u, 0u, 0u, 0u);
                    }
                mbar_wait(&bars[LB_TFULL + acc], acc_ph, wctx, LB_TFULL + acc);
                tc_fence_after();
                const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * L_BN + half_n * (L_BN / 2);
                // ---- pass 1: x = acc + bias + residual back into tensor memory; this thread's statistics over 128 columns
                float cnt = 0.f, mean = 0.f, m2 = 0.f;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {                          // 32 columns at a time
                    uint32_t r[32];
                    tmem_ld32(t_row + ch * 32, r);
                    tc_wait_ld();
                    float2 sum2 = pk2(0.f, 0.f);
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int col = colbase + ch * 32 + 8 * g;
                        const __half2* rh = reinterpret_cast<const __half2*>(&res[ch >> 1][(ch & 1) * 4 + g]);
                        uint4 bu = make_uint4(0u, 0u, 0u, 0u);
                        if (bias != nullptr) bu = __ldg(reinterpret_cast<const uint4*>(bias + col));
                        const __half2* bh = reinterpret_cast<const __half2*>(&bu);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 fr = __half22float2(rh[j]), fb = __half22float2(bh[j]);
                            float2 v = pk2(__uint_as_float(r[8 * g + 2 * j]), __uint_as_float(r[8 * g + 2 * j + 1]));
                            v = add2(add2(v, pk2(fb.x, fb.y)), pk2(fr.x, fr.y));
                            sum2 = add2(sum2, v);
                            r[8 * g + 2 * j] = __float_as_uint(v.x);
                            r[8 * g + 2 * j + 1] = __float_as_uint(v.y);
                        }
                    }
                    tmem_st32(t_row + ch * 32, r);
                    const float mean_c = (sum2.x + sum2.y) * (1.0f / 32.0f);
                    const float2 nm = pk2(-mean_c, -mean_c);
                    float2 sq2 = pk2(0.f, 0.f);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float2 d = add2(pk2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), nm);
                        sq2 = fma2(d, d, sq2);
                    }
                    if (ch == 0) { cnt = 32.f; mean = mean_c; m2 = sq2.x + sq2.y; }
                    else merge_stats(cnt, mean, m2, 32.f, mean_c, sq2.x + sq2.y);
                }
                tc_wait_st();
                // this thread's partial goes to every block of the cluster (its own included); once the whole warp has stored,
                // one lane reports to each block (its release-arrive follows the warp barrier, so it covers the other lanes' stores)
                {
                    float2* slot = partials + ((acc * L_MAX_CLUSTER + rank) * 2 + half_n) * L_BM + lrow;
                    const uint32_t local_slot = smem_u32(slot), local_bar = smem_u32(&bars[LB_PART + acc]);
                    for (int d = 0; d < cluster_size; ++d) st_cluster_f32x2(map_to_rank(local_slot, static_cast<uint32_t>(d)), mean, m2);
                    __syncwarp();
                    if (lane < cluster_size) remote_arrive(map_to_rank(local_bar, static_cast<uint32_t>(lane)));
                }
                mbar_wait_cluster(&bars[LB_PART + acc], acc_ph, wctx, LB_PART + acc);
                // ---- the row's statistics from the 2 * cluster_size partials
                {
                    const float2* base = partials + (acc * L_MAX_CLUSTER * 2) * L_BM + lrow;
                    const float2 p0 = base[0];
                    cnt = 128.f; mean = p0.x; m2 = p0.y;
                    for (int i = 1; i < 2 * cluster_size; ++i) {
                        const float2 pi = base[i * L_BM];
                        merge_stats(cnt, mean, m2, 128.f, pi.x, pi.y);
                    }
                }
                const float rstd = 1.0f / sqrtf(m2 * inv_n + eps);
                const float2 rstd2 = pk2(rstd, rstd), shift2 = pk2(-mean * rstd, -mean * rstd);
                // ---- pass 2: normalise, scale, shift, store (32 columns per tensor-memory load, 64 per TMA store)
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    const int col0 = colbase + ch * 64;
                    if (lane == 0) tma_store_wait_read();                 // the slab's previous store has been read out
                    __syncwarp();
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        uint32_t r[32];
                        tmem_ld32(t_row + ch * 64 + hh * 32, r);
                        tc_wait_ld();
                        if (ch == 1 && hh == 1) {
                            // the accumulator has been read for the last time: hand it back to the MMA warp
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&bars[LB_TEMPTY + acc]);
                        }
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const int col = col0 + hh * 32 + 8 * g;
                            uint4 gu = make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u), bu = make_uint4(0u, 0u, 0u, 0u);   // 1.0, 0.0
                            if (gamma != nullptr) gu = __ldg(reinterpret_cast<const uint4*>(gamma + col));
                            if (beta != nullptr) bu = __ldg(reinterpret_cast<const uint4*>(beta + col));
                            const __half2* gh = reinterpret_cast<const __half2*>(&gu);
                            const __half2* bh = reinterpret_cast<const __half2*>(&bu);
                            uint32_t o[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 fg = __half22float2(gh[j]), fb = __half22float2(bh[j]);
                                float2 v = fma2(pk2(__uint_as_float(r[8 * g + 2 * j]), __uint_as_float(r[8 * g + 2 * j + 1])), rstd2, shift2);
                                v = fma2(v, pk2(fg.x, fg.y), pk2(fb.x, fb.y));
                                o[j] = pack_half2(v.x, v.y);
                            }
                            *reinterpret_cast<uint4*>(slab + lane * 128 + (((hh * 4 + g) ^ (lane & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && row0 < m) {
                        tma_store_2d(&map_c, slab, col0, row0);           // rows beyond the matrix are clipped by the tensor map
                        tma_store_commit();
                    }
                }
            }
            if (lane == 0) tma_store_wait_all();
        }
    }
    // no block leaves while a peer may still write its partials table or signal one of its barriers
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == L_EPI_WARPS + 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, L_TMEM_COLS);
    }
}

}  // namespace
}  // namespace stof

using namespace stof;

// Declared in include/stof_b200.h.  Shapes the fused kernel does not cover (N not a multiple of 256, or beyond 1024) run as the
// GEMM with the bias + residual epilogue followed by the row LayerNorm kernel in place - and so do long contractions
// (K > 2048): there the main loop decides, the two-block GEMM kernel's is faster than this kernel's one-block main loop by more
// than the separate LayerNorm pass costs (measured at T = 65536: K = 4096, N = 1024: 455 us against 504 us fused; K = 1024,
// N = 1024: 180 us either way; K = 768, N = 768: 161 us against 148 us fused).  STOF_B200_GEMM_LN=fused / split overrides.
extern "C" int stof_gemm_bias_residual_layernorm(const void* a, long long lda, const void* w, long long ldw, const void* bias,
                                                 const void* residual, long long ldr, const void* gamma, const void* beta, float eps,
                                                 void* c, long long ldc, int m, int n, int k, int* status_dev, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    STOF_REQUIRE(a && w && c, "gemm+layernorm: null operand");
    STOF_REQUIRE(m >= 0 && n > 0 && k > 0, "gemm+layernorm: bad shape m=%d n=%d k=%d", m, n, k);
    STOF_REQUIRE(n % 8 == 0 && k % 8 == 0, "gemm+layernorm: n=%d and k=%d must be multiples of 8", n, k);
    STOF_REQUIRE(lda % 8 == 0 && ldw % 8 == 0 && ldc % 8 == 0, "gemm+layernorm: leading dimensions must be multiples of 8 elements");
    STOF_REQUIRE(lda >= k && ldw >= n && ldc >= n, "gemm+layernorm: leading dimension smaller than the row length");
    STOF_REQUIRE(aligned16(a) && aligned16(w) && aligned16(c) && aligned16(bias) && aligned16(residual) && aligned16(gamma) && aligned16(beta),
                 "gemm+layernorm: pointers must be 16-byte aligned");
    STOF_REQUIRE(!residual || (ldr % 8 == 0 && ldr >= n), "gemm+layernorm: residual row stride must be a multiple of 8, >= n");
    if (m == 0) return STOF_OK;
    static const int mode = [] {
        const char* e = std::getenv("STOF_B200_GEMM_LN");
        return e == nullptr ? 0 : (e[0] == 'f' ? 1 : (e[0] == 's' ? 2 : 0));
    }();
    const bool fused = n % L_BN == 0 && n / L_BN <= L_MAX_CLUSTER && mode != 2 && (mode == 1 || k <= 2048);
    if (!fused) {
        int rc = residual ? stof_gemm_bias_act(a, lda, w, ldw, bias, residual, ldr, c, ldc, m, n, k, STOF_EPI_BIAS_RESIDUAL, status_dev, stream_)
                          : stof_gemm_bias_act(a, lda, w, ldw, bias, nullptr, 0, c, ldc, m, n, k, STOF_EPI_BIAS, status_dev, stream_);
        if (rc != STOF_OK) return rc;
        return stof_bias_residual_layernorm(c, ldc, nullptr, nullptr, 0, gamma, beta, eps, c, ldc, m, n, status_dev, stream_);
    }
    CUtensorMap ma, mw, mc;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m)};
        const uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
        const uint32_t box[2] = {L_BK, L_BM};
        if (int rc = make_tensor_map_f16(&ma, a, 2, dims, strides, box)) return rc;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(k)};
        const uint64_t strides[1] = {static_cast<uint64_t>(ldw) * 2};
        const uint32_t box[2] = {64, L_BK};
        if (int rc = make_tensor_map_f16(&mw, w, 2, dims, strides, box)) return rc;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(m)};
        const uint64_t strides[1] = {static_cast<uint64_t>(ldc) * 2};
        const uint32_t box[2] = {64, 32};
        if (int rc = make_tensor_map_f16(&mc, c, 2, dims, strides, box)) return rc;
    }
    static std::atomic<bool> configured[64];     // per device; host threads may race here, every one of them stores the same value
    int dev = 0;
    STOF_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        STOF_CUDA(cudaFuncSetAttribute(gemm_ln_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(L_SMEM)));
        configured[dev] = true;
    }
    const int cluster = n / L_BN;
    const int tiles_m = (m + L_BM - 1) / L_BM;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((sm_count() / cluster) * cluster));
    cfg.blockDim = dim3(L_THREADS);
    cfg.dynamicSmemBytes = L_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // persistent: exactly as many clusters as the GPU keeps resident at once (the SMs of a cluster lie in one processing
    // cluster of the chip, so fewer than SMs / cluster size may fit), cached per device and cluster size
    static std::atomic<int> resident[64][L_MAX_CLUSTER + 1];
    int clusters = (dev >= 0 && dev < 64) ? resident[dev][cluster].load() : 0;
    if (clusters == 0) {
        STOF_CUDA(cudaOccupancyMaxActiveClusters(&clusters, gemm_ln_kernel, &cfg));
        if (clusters < 1) {
            set_error("gemm+layernorm: no cluster of %d thread blocks fits on this GPU", cluster);
            return STOF_E_LIMIT;
        }
        if (dev >= 0 && dev < 64) resident[dev][cluster].store(clusters);
    }
    if (clusters > tiles_m) clusters = tiles_m;
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * cluster));
    STOF_CUDA(cudaLaunchKernelEx(&cfg, gemm_ln_kernel, ma, mw, mc, static_cast<const __half*>(bias), static_cast<const __half*>(residual), ldr,
                                 static_cast<const __half*>(gamma), static_cast<const __half*>(beta), eps, m, n, k, cluster, status_dev));
    return STOF_OK;
}
