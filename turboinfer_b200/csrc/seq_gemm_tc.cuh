// seq_gemm_tc.cuh -- bf16 x bf16 -> fp32 GEMM on the 5th-generation tensor cores for the prompt side of the layered sequence
// engine:  C[M, N] = epi(A[M, K] . W[N, K]^T), A = bf16 activations (row-major), W = bf16 weights as stored ([out, in]).
// Both operands are K-major, so both are fetched with plain 2-D TMA boxes (64 elements = 128 bytes x 128 rows, SWIZZLE_128B;
// rows and k beyond the tensor are zero-filled by the copy engine, so no operand is padded in memory).
//
//   CTA tile      128 rows x 128 columns, k-steps of 64 elements, 3-stage ring of 32 KiB (two CTAs fit an SM: one CTA's
//                 epilogue overlaps the other's main loop); 128 TMEM columns of fp32 accumulators
//   warp 0        producer (one lane): TMA loads of the A and W boxes, completion on the stage's `full` barrier
//   warp 1        TMEM allocation; one lane issues tcgen05.mma kind::f16 (M 128, N 128, K 16), four per stage;
//                 tcgen05.commit frees the stage / publishes the accumulators
//   warps 2..5    epilogue: tcgen05.ld 32x32b (lane = row), optional activation / scale, 64-byte stores per lane
// Every wait is bounded: a wait that runs out sets *err and the roles fall through to the common exit, where TMEM is freed.
#pragma once
#include "gemm_tc.cuh"
#include "seq_kernels.cuh"

namespace tib {
namespace seq {

constexpr int kSgBM = 128, kSgBN = 128, kSgBK = 64;      // BK in bf16 elements (128 bytes)
constexpr int kSgStages = 3;
constexpr int kSgThreads = 192;
constexpr int kSgTileBytes = kSgBM * kSgBK * 2;          // 16 KiB
constexpr int kSgStageBytes = 2 * kSgTileBytes;
constexpr size_t kSgSmemBytes = (size_t)kSgStages * kSgStageBytes + 1024 /*align*/ + 256 /*barriers*/;

struct TcArgs {
    int M, N, K;
    float* C;
    int ldc;
    int epi;
    float alpha, beta;
    int* err;   // set to 1 when a wait ran out
};

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* err) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > 2000000000LL) {   // about a second
            atomicExch(err, 1);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D fp32, A and B bf16, both K-major
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__global__ void __launch_bounds__(kSgThreads, 2)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const TcArgs g) {
    extern __shared__ uint8_t tsm_raw[];
    const uint32_t base = (smem_u32(tsm_raw) + 1023u) & ~1023u;
    uint8_t* tiles = tsm_raw + (base - smem_u32(tsm_raw));
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)kSgStages * kSgStageBytes);
    uint64_t* empty = full + kSgStages;
    uint64_t* tmem_full = empty + kSgStages;
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tmem_full + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = blockIdx.x, mb = blockIdx.y;
    const int KB = (g.K + kSgBK - 1) / kSgBK;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kSgStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        mbar_init(tmem_full, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr)), "n"(kSgBN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_ptr;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < KB; ++kb) {
                const int st = kb % kSgStages, use = kb / kSgStages;
                if (use > 0 && !mbar_wait_bounded(&empty[st], (use - 1) & 1, g.err)) break;
                mbar_arrive_expect_tx(&full[st], kSgStageBytes);
                uint8_t* sbase = tiles + (size_t)st * kSgStageBytes;
                tma_load_2d(sbase, &map_a, kb * kSgBK, mb * kSgBM, &full[st]);
                tma_load_2d(sbase + kSgTileBytes, &map_w, kb * kSgBK, nb * kSgBN, &full[st]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(kSgBM, kSgBN);
            bool ok = true;
            for (int kb = 0; kb < KB && ok; ++kb) {
                const int st = kb % kSgStages, use = kb / kSgStages;
                ok = mbar_wait_bounded(&full[st], use & 1, g.err);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sbase = base + st * kSgStageBytes;
#pragma unroll
                for (int k4 = 0; k4 < kSgBK / 16; ++k4) {
                    const uint64_t adesc = umma_desc_sw128(sbase + k4 * 32);
                    const uint64_t bdesc = umma_desc_sw128(sbase + kSgTileBytes + k4 * 32);
                    tc_mma_bf16(tmem, adesc, bdesc, idesc, (kb | k4) != 0 ? 1u : 0u);
                }
                tc_commit(&empty[st]);
            }
            tc_commit(tmem_full);   // also on the failure path: the epilogue warps must not wait for ever
        }
    } else {
        const bool ok = mbar_wait_bounded(tmem_full, 0, g.err);
        tc_fence_after();
        const int q = warp & 3;
        const int row = mb * kSgBM + q * 32 + lane;
        const bool row_ok = ok && row < g.M && *reinterpret_cast<volatile int*>(g.err) == 0;
        for (int c0 = 0; c0 < kSgBN; c0 += 16) {
            uint32_t a[16];
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]),
                  "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15])
                : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row_ok) {
                const int nbase = nb * kSgBN + c0;
                float* crow = g.C + (size_t)row * g.ldc;
                if ((g.ldc & 3) == 0 && nbase + 16 <= g.N && (reinterpret_cast<uintptr_t>(g.C) & 15) == 0) {
#pragma unroll
                    for (int i = 0; i < 16; i += 4) {
                        float4 v = make_float4(epi_apply(__uint_as_float(a[i]), g.epi, g.alpha, g.beta), epi_apply(__uint_as_float(a[i + 1]), g.epi, g.alpha, g.beta),
                                               epi_apply(__uint_as_float(a[i + 2]), g.epi, g.alpha, g.beta), epi_apply(__uint_as_float(a[i + 3]), g.epi, g.alpha, g.beta));
                        *reinterpret_cast<float4*>(crow + nbase + i) = v;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (nbase + i < g.N) crow[nbase + i] = epi_apply(__uint_as_float(a[i]), g.epi, g.alpha, g.beta);
                }
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kSgBN) : "memory");
    }
}

}  // namespace seq
}  // namespace tib
