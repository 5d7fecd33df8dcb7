// y = LayerNorm(x + bias + residual) * gamma + beta over rows of fp16, fp32 statistics (HBM-bound).
//
// One warp per row, persistent over rows.  A row is read once (through a shared-memory ring fed by bulk copies, two further
// rows of the warp in flight), held in registers as packed fp32 pairs, reduced with warp shuffles (mean, then the centred
// sum of squares, biased variance as src/triton_template/add_layernorm.py:33-55 and F.layer_norm do), and written once
// with 128-bit stores; gamma and beta of a lane's columns stay in registers across rows.  Rows longer than 2048 elements are re-read from cache for the second and third sweep
// instead of being held in registers.
#include "stof_host.h"
#include "stof_ptx.cuh"

#include <cuda_fp16.h>

namespace stof {
namespace {

constexpr int LN_WARPS = 8;
constexpr int LN_BLOCKS_PER_SM = 4;
constexpr int LN_STAGES = 3;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void load8(const __half* p, float (&f)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__device__ __forceinline__ void add8(const __half* p, float (&f)[8]) {
    float t[8];
    load8(p, t);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] += t[i];
}

__device__ __forceinline__ void store8(__half* p, const float (&f)[8]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
}

// NCHUNK: 16-byte chunks held per lane (hidden <= NCHUNK * 256); NCHUNK == 0 selects the re-reading variant.
// Persistent: each warp walks rows warp, warp + W, ...  Rows (and residual rows) arrive through a per-warp ring of
// LN_STAGES shared-memory buffers filled by 1-D bulk copies, so that two further rows per warp are always in flight and
// the kernel keeps enough bytes outstanding to cover the HBM latency without spending registers on it.
template <int NCHUNK>
__global__ void __launch_bounds__(LN_WARPS * 32)
layernorm_kernel(const __half* x, long long ldx, const __half* __restrict__ bias, const __half* __restrict__ residual,
                 long long ldr, const __half* __restrict__ gamma, const __half* __restrict__ beta, float eps, __half* y,
                 long long ldy, int rows, int hidden, int* status) {
    extern __shared__ __align__(128) unsigned char ln_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps_total = gridDim.x * LN_WARPS;
    int row = blockIdx.x * LN_WARPS + warp;
    if (row >= rows) return;
    const int nchunks = hidden >> 3;
    const float inv_n = 1.0f / static_cast<float>(hidden);

    if constexpr (NCHUNK > 0) {
        const uint32_t row_bytes = static_cast<uint32_t>(hidden) * 2u;
        const uint32_t slot_bytes = residual ? 2u * row_bytes : row_bytes;
        uint64_t* bars = reinterpret_cast<uint64_t*>(ln_smem) + warp * LN_STAGES;
        unsigned char* ring = ln_smem + LN_WARPS * LN_STAGES * 8 + static_cast<size_t>(warp) * LN_STAGES * slot_bytes;
        if (lane == 0) {
            for (int s = 0; s < LN_STAGES; ++s) mbar_init(&bars[s], 1);
            fence_mbar_init();
        }
        __syncwarp();
        auto issue = [&](int r_logical, int s) {         // lane 0 only
            const int r = rows - 1 - r_logical;          // rows are visited from the last to the first (see the launcher)
            unsigned char* dst = ring + static_cast<size_t>(s) * slot_bytes;
            mbar_arrive_expect_tx(&bars[s], slot_bytes);
            bulk_load_1d(dst, x + static_cast<size_t>(r) * ldx, row_bytes, &bars[s]);
            if (residual) bulk_load_1d(dst + row_bytes, residual + static_cast<size_t>(r) * ldr, row_bytes, &bars[s]);
        };
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < LN_STAGES - 1; ++s)
                if (row + s * warps_total < rows) issue(row + s * warps_total, s);
        }
        // 8 halves -> 4 packed fp32 pairs
        auto unpack2 = [](const uint4& u, float2 (&f)[4]) {
            const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int i = 0; i < 4; ++i) f[i] = __half22float2(h[i]);
        };
        // gamma and beta of this lane's columns stay in registers as fp32 pairs for every row the warp processes
        // (rows up to 1024 columns; longer rows convert them per row to bound the register count)
        constexpr bool AFFINE_IN_REGS = NCHUNK <= 4;
        float2 g2[AFFINE_IN_REGS ? NCHUNK : 1][4], b2[AFFINE_IN_REGS ? NCHUNK : 1][4];
        if constexpr (AFFINE_IN_REGS) {
#pragma unroll
            for (int i = 0; i < NCHUNK; ++i) {
                const int c = lane + 32 * i;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    g2[i][j] = make_float2(1.0f, 1.0f);
                    b2[i][j] = make_float2(0.0f, 0.0f);
                }
                if (c < nchunks) {
                    if (gamma) unpack2(__ldg(reinterpret_cast<const uint4*>(gamma + 8 * c)), g2[i]);
                    if (beta) unpack2(__ldg(reinterpret_cast<const uint4*>(beta + 8 * c)), b2[i]);
                }
            }
        }
        for (int it = 0; row < rows; row += warps_total, ++it) {
            const int s = it % LN_STAGES;
            const uint32_t parity = static_cast<uint32_t>((it / LN_STAGES) & 1);
            // completes with the copy (no partner thread involved); bounded all the same by a cycle budget: a warp whose copy
            // never lands reports it and leaves its remaining rows unwritten instead of normalising stale shared memory
            if (!__all_sync(0xffffffffu, mbar_wait_budget(&bars[s], parity))) {
                if (lane == 0 && status) atomicCAS(status, 0, (s << 8) | STATUS_WAIT_TIMEOUT);
                break;
            }
            const unsigned char* src = ring + static_cast<size_t>(s) * slot_bytes;
            float2 v[NCHUNK][4];
            float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < NCHUNK; ++i) {
                const int c = lane + 32 * i;
#pragma unroll
                for (int j = 0; j < 4; ++j) v[i][j] = make_float2(0.f, 0.f);
                if (c < nchunks) {
                    unpack2(*reinterpret_cast<const uint4*>(src + 16 * c), v[i]);
                    float2 t[4];
                    if (residual) {
                        unpack2(*reinterpret_cast<const uint4*>(src + row_bytes + 16 * c), t);
#pragma unroll
                        for (int j = 0; j < 4; ++j) v[i][j] = add2(v[i][j], t[j]);
                    }
                    if (bias) {
                        unpack2(__ldg(reinterpret_cast<const uint4*>(bias + 8 * c)), t);
#pragma unroll
                        for (int j = 0; j < 4; ++j) v[i][j] = add2(v[i][j], t[j]);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) sum2 = add2(sum2, v[i][j]);
                }
            }
            // this slot is read out: refill the slot that was consumed one row ago with the row LN_STAGES - 1 ahead
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                const int ahead = row + (LN_STAGES - 1) * warps_total;
                if (ahead < rows) issue(ahead, (it + LN_STAGES - 1) % LN_STAGES);
            }
            const float mean = warp_sum(sum2.x + sum2.y) * inv_n;
            const float2 nmean2 = make_float2(-mean, -mean);
            float2 sq2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < NCHUNK; ++i) {
                if (lane + 32 * i < nchunks) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        v[i][j] = add2(v[i][j], nmean2);                  // centred value, kept for the output pass
                        sq2 = fma2(v[i][j], v[i][j], sq2);
                    }
                }
            }
            const float rstd = 1.0f / sqrtf(warp_sum(sq2.x + sq2.y) * inv_n + eps);
            const float2 rstd2 = make_float2(rstd, rstd);
            __half* yr = y + static_cast<size_t>(rows - 1 - row) * ldy;
#pragma unroll
            for (int i = 0; i < NCHUNK; ++i) {
                const int c = lane + 32 * i;
                if (c < nchunks) {
                    float2 gg[4], bb[4];
                    if constexpr (!AFFINE_IN_REGS) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            gg[j] = make_float2(1.0f, 1.0f);
                            bb[j] = make_float2(0.0f, 0.0f);
                        }
                        if (gamma) unpack2(__ldg(reinterpret_cast<const uint4*>(gamma + 8 * c)), gg);
                        if (beta) unpack2(__ldg(reinterpret_cast<const uint4*>(beta + 8 * c)), bb);
                    }
                    uint4 u;
                    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 g = AFFINE_IN_REGS ? g2[AFFINE_IN_REGS ? i : 0][j] : gg[j];
                        const float2 bt = AFFINE_IN_REGS ? b2[AFFINE_IN_REGS ? i : 0][j] : bb[j];
                        const float2 o = fma2(mul2(v[i][j], rstd2), g, bt);
                        h[j] = __floats2half2_rn(o.x, o.y);
                    }
                    *reinterpret_cast<uint4*>(yr + 8 * c) = u;
                }
            }
        }
    } else {
        for (; row < rows; row += warps_total) {
            const __half* xr = x + static_cast<size_t>(rows - 1 - row) * ldx;
            const __half* rr = residual ? residual + static_cast<size_t>(rows - 1 - row) * ldr : nullptr;
            __half* yr = y + static_cast<size_t>(rows - 1 - row) * ldy;
            float sum = 0.f;
            for (int c = lane; c < nchunks; c += 32) {
                float t[8];
                load8(xr + 8 * c, t);
                if (bias) add8(bias + 8 * c, t);
                if (rr) add8(rr + 8 * c, t);
#pragma unroll
                for (int j = 0; j < 8; ++j) sum += t[j];
            }
            const float mean = warp_sum(sum) * inv_n;
            float sq = 0.f;
            for (int c = lane; c < nchunks; c += 32) {
                float t[8];
                load8(xr + 8 * c, t);
                if (bias) add8(bias + 8 * c, t);
                if (rr) add8(rr + 8 * c, t);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float d = t[j] - mean;
                    sq += d * d;
                }
            }
            const float rstd = 1.0f / sqrtf(warp_sum(sq) * inv_n + eps);
            for (int c = lane; c < nchunks; c += 32) {
                float t[8], g[8], b[8];
                load8(xr + 8 * c, t);
                if (bias) add8(bias + 8 * c, t);
                if (rr) add8(rr + 8 * c, t);
                if (gamma) load8(gamma + 8 * c, g);
                if (beta) load8(beta + 8 * c, b);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float o = (t[j] - mean) * rstd;
                    if (gamma) o *= g[j];
                    if (beta) o += b[j];
                    t[j] = o;
                }
                store8(yr + 8 * c, t);
            }
        }
    }
}

}  // namespace
}  // namespace stof

using namespace stof;

extern "C" int stof_bias_residual_layernorm(const void* x, long long ldx, const void* bias, const void* residual, long long ldr,
                                            const void* gamma, const void* beta, float eps, void* y, long long ldy, int rows, int hidden,
                                            int* status_dev, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    STOF_REQUIRE(x && y, "layernorm: null x or y");
    STOF_REQUIRE(rows >= 0 && hidden > 0, "layernorm: bad shape (%d, %d)", rows, hidden);
    STOF_REQUIRE(hidden % 8 == 0, "layernorm: hidden %d must be a multiple of 8", hidden);
    if (hidden > 8192) {
        set_error("layernorm: hidden %d beyond the maximum of 8192", hidden);
        return STOF_E_LIMIT;
    }
    STOF_REQUIRE(ldx % 8 == 0 && ldy % 8 == 0 && (!residual || ldr % 8 == 0), "layernorm: row strides must be multiples of 8 elements");
    STOF_REQUIRE(ldx >= hidden && ldy >= hidden && (!residual || ldr >= hidden), "layernorm: row stride smaller than hidden");
    STOF_REQUIRE(aligned16(x) && aligned16(y) && aligned16(bias) && aligned16(residual) && aligned16(gamma) && aligned16(beta),
                 "layernorm: pointers must be 16-byte aligned");
    if (rows == 0) return STOF_OK;
    const dim3 block(LN_WARPS * 32);
    const __half *xp = static_cast<const __half*>(x), *bp = static_cast<const __half*>(bias), *rp = static_cast<const __half*>(residual),
                 *gp = static_cast<const __half*>(gamma), *tp = static_cast<const __half*>(beta);
    __half* yp = static_cast<__half*>(y);
    const size_t ring_smem = hidden <= 2048 ? static_cast<size_t>(LN_WARPS) * LN_STAGES * (8 + static_cast<size_t>(hidden) * 2 * (residual ? 2 : 1)) : 0;
    // persistent grid: as many blocks as are resident at once (registers and the ring decide), never more than the rows need.
    // The kernel visits the rows from the last to the first: the producer of x (a GEMM walking its tiles upwards) wrote the
    // last rows most recently, so they are the ones still in L2, and the rows this kernel writes last are the first a
    // following GEMM reads (0.3 % of a BERT-large forward, measured)
#define STOF_LN_LAUNCH(N)                                                                                                           \
    do {                                                                                                                            \
        if (ring_smem > 48 * 1024)                                                                                                  \
            STOF_CUDA(cudaFuncSetAttribute(layernorm_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ring_smem))); \
        int per_sm = 0;                                                                                                             \
        STOF_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, layernorm_kernel<N>, LN_WARPS * 32, ring_smem));           \
        if (per_sm < 1) per_sm = 1;                                                                                                 \
        if (per_sm > LN_BLOCKS_PER_SM) per_sm = LN_BLOCKS_PER_SM;                                                                   \
        int blocks = (rows + LN_WARPS - 1) / LN_WARPS;                                                                              \
        if (blocks > sm_count() * per_sm) blocks = sm_count() * per_sm;                                                             \
        layernorm_kernel<N><<<dim3(blocks), block, ring_smem, stream>>>(xp, ldx, bp, rp, ldr, gp, tp, eps, yp, ldy, rows, hidden, status_dev);   \
    } while (0)
    if (hidden <= 256) STOF_LN_LAUNCH(1);
    else if (hidden <= 512) STOF_LN_LAUNCH(2);
    else if (hidden <= 768) STOF_LN_LAUNCH(3);
    else if (hidden <= 1024) STOF_LN_LAUNCH(4);
    else if (hidden <= 2048) STOF_LN_LAUNCH(8);
    else STOF_LN_LAUNCH(0);
#undef STOF_LN_LAUNCH
    STOF_CUDA(cudaGetLastError());
    return STOF_OK;
}
