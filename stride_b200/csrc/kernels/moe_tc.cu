// The experts' products of a routed feed-forward on the fifth-generation tensor cores, for steps of many rows
// (portions of prompts):
//   C[p, :] = act(A[p, :] W[e(p)]^T)   for the rows p of every expert e, rows lying expert by expert (`offsets`).
//
// One CTA computes a 128 x BLOCK_N tile: 128 rows of one expert, BLOCK_N output features of that expert. The row
// tile `blockIdx.y` is found from `offsets` on the device (nothing returns to the host). A producer thread streams
// 128 x 64 tiles of A and BLOCK_N x 64 tiles of the stacked weights [experts * N, K] into a ring of shared-memory
// stages with TMA (128-byte swizzle, completion on an mbarrier); one thread issues tcgen05.mma with the accumulator
// in tensor memory and frees each stage with tcgen05.commit; four warps read the accumulator back with tcgen05.ld, a
// row a thread, apply the activation and store. Rows of the tile past the expert's last row and features past its
// last feature are computed from whatever lies there (the next expert's rows, zeros past the end) and not stored.
// Two CTAs fit one SM, so one tile's epilogue runs under the other's products.
//
// act 0: none; 1: the square of the positive part; 2: the rows of W come as (gate, up) pairs, row 2i beside row
// 2i + 1, and the tile leaves g' sigmoid(alpha g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit), N / 2 wide;
// 3: the same pairs, and the tile leaves g sigmoid(g) u.
//
// gather_rows lays the rows of the step's tokens out expert by expert first (xs[p] = x[perm[p]]), so that the first
// product's A operand is one matrix a tensor map can describe; the second product's input is in that order already.
//
// Every wait on an mbarrier is bounded by a clock; a wait that runs out sets *status and the CTA winds down
// (tensor memory is freed on every path).
#include "tcgen05.cuh"

namespace stride {
namespace tc {

constexpr int kGroupM = 128;
constexpr int kGroupK = 64;              // 64 bf16 = one 128-byte swizzle row
constexpr int kGroupThreads = 192;       // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue

__device__ __forceinline__ float act_clamped(float g, float u, float limit, float alpha) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}

__device__ __forceinline__ void store4(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float* v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&a);
    u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ void store1(float* p, float v) { *p = v; }
__device__ __forceinline__ void store1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int BLOCK_N, int STAGES, typename OutT>
__global__ void __launch_bounds__(kGroupThreads, 2)
grouped_gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                        const int32_t* __restrict__ offsets, int experts, OutT* __restrict__ C, int ldc, int N, int K, int act,
                        float limit, float alpha, int vec_ok, int* __restrict__ status) {
    constexpr int A_BYTES = kGroupM * kGroupK * 2;
    constexpr int W_BYTES = BLOCK_N * kGroupK * 2;
    constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
    constexpr uint32_t TMEM_COLS = BLOCK_N < 32 ? 32 : BLOCK_N;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_base_slot;

    pdl_trigger();
    pdl_wait();                  // the plan (offsets) and the rows come from the kernels before this one
    // which expert's rows this tile holds: uniform over the CTA, so everybody leaves together when there is none
    int tile = blockIdx.y, e = 0, m0 = 0, m_end = 0;
    for (; e < experts; ++e) {
        const int lo = offsets[e], hi = offsets[e + 1];
        const int tiles = (hi - lo + kGroupM - 1) / kGroupM;
        if (tile < tiles) {
            m0 = lo + tile * kGroupM;
            m_end = hi;
            break;
        }
        tile -= tiles;
    }
    if (e >= experts) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BLOCK_N;
    const int num_kb = (K + kGroupK - 1) / kGroupK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&done_bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {
            const int w_row = e * N + n0;
            for (int i = 0; i < num_kb; ++i) {
                const int s = i % STAGES;
                if (i >= STAGES && !mbar_wait(smem_u32(&empty_bar[s]), ((i / STAGES) & 1) ^ 1, status, 11)) break;
                const uint32_t bar = smem_u32(&full_bar[s]);
                mbar_expect_tx(bar, STAGE_BYTES);
                const uint32_t a_dst = smem_u32(smem + s * STAGE_BYTES);
                tma_load_2d(a_dst, &map_a, bar, i * kGroupK, m0);
                tma_load_2d(a_dst + A_BYTES, &map_w, bar, i * kGroupK, w_row);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(kGroupM, BLOCK_N, false);
            for (int i = 0; i < num_kb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(smem_u32(&full_bar[s]), (i / STAGES) & 1, status, 12)) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
                const uint64_t a_desc = smem_desc_sw128(a_addr), w_desc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                for (int k = 0; k < kGroupK / 16; ++k)      // 16 elements along K inside the swizzled row: +32 bytes
                    umma_bf16(tmem_base, a_desc + 2 * k, w_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(smem_u32(&empty_bar[s]));
            }
            umma_commit(smem_u32(&done_bar));
        }
        __syncwarp();
    } else {
        // warps 2..5 own the lane quadrants 2, 3, 0, 1 of tensor memory; a thread holds one row of the tile
        const int quad = warp & 3;
        const int m = m0 + quad * 32 + lane;
        const bool ok = mbar_wait(smem_u32(&done_bar), 0, status, 13);
        tc_fence_after();
        if (ok) {
            const int width = act >= 2 ? N / 2 : N;
            OutT* crow = C + static_cast<size_t>(m) * ldc;
#pragma unroll 1
            for (int c0 = 0; c0 < BLOCK_N; c0 += 32) {
                if (n0 + c0 >= N) break;                       // uniform over the warp
                float v[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + c0, v);
                if (m >= m_end) continue;
                if (act >= 2) {
                    const int col = (n0 + c0) / 2;
                    float r[16];
                    if (act == 3) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) r[j] = v[2 * j] / (1.f + expf(-v[2 * j])) * v[2 * j + 1];
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) r[j] = act_clamped(v[2 * j], v[2 * j + 1], limit, alpha);
                    }
                    if (vec_ok && col + 16 <= width) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4) store4(crow + col + j, r + j);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (col + j < width) store1(crow + col + j, r[j]);
                    }
                } else {
                    if (act == 1) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float p = fmaxf(v[j], 0.f);
                            v[j] = p * p;
                        }
                    }
                    const int col = n0 + c0;
                    if (vec_ok && col + 32 <= width) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) store4(crow + col + j, v + j);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col + j < width) store1(crow + col + j, v[j]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// xs[p, :] = x[perm[p], :] for the rows p below offsets[experts]; 16 bytes a thread.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ x, int ldx16, const int32_t* __restrict__ perm, const int32_t* __restrict__ offsets, int experts,
                   uint4* __restrict__ xs, int row16, int max_rows) {
    pdl_trigger();
    pdl_wait();
    const int total = min(offsets[experts], max_rows);
    for (int p = blockIdx.x; p < total; p += gridDim.x) {
        const int src = perm[p];
        if (src < 0) continue;
        const uint4* from = x + static_cast<size_t>(src) * ldx16;
        uint4* to = xs + static_cast<size_t>(p) * row16;
        for (int c = threadIdx.x; c < row16; c += blockDim.x) to[c] = from[c];
    }
}

template <typename OutT>
int launch_grouped(const CUtensorMap* map_a, const CUtensorMap* map_w, const int32_t* offsets, int experts, OutT* C, int ldc, int max_rows,
                   int N, int K, int act, float limit, float alpha, int vec_ok, int* status, cudaStream_t stream) {
    constexpr int BLOCK_N = 128, STAGES = 3;
    constexpr int smem = STAGES * (kGroupM * kGroupK * 2 + BLOCK_N * kGroupK * 2) + 1024;
    static bool configured[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return STRIDE_BAD_ARGUMENT;
    auto kernel = grouped_gemm_tc5_kernel<BLOCK_N, STAGES, OutT>;
    if (!configured[device]) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) return static_cast<int>(err);
        configured[device] = true;
    }
    const int max_tiles = (max_rows + kGroupM - 1) / kGroupM + experts;       // no expert has more than one ragged tile
    if (max_tiles > 65535) return STRIDE_UNSUPPORTED;
    const dim3 grid((N + BLOCK_N - 1) / BLOCK_N, max_tiles);
    stride::launch(kernel, grid, dim3(kGroupThreads), smem, stream, *map_a, *map_w, offsets, experts, C, ldc, N, K, act, limit, alpha, vec_ok,
                   status);
    return STRIDE_LAUNCH_STATUS();
}

}  // namespace tc
}  // namespace stride

using namespace stride;

extern "C" {

// C[p] = act(A[p] @ W[e(p)]^T) for rows lying expert by expert. A: [max_rows, K] bf16 with row stride lda, W: [experts, N, K] bf16,
// C: [max_rows, N] (N / 2 with act 2 and 3), bf16 or float32. Returns -2 for what it does not take (K or lda not a multiple of
// 8, unaligned operands); the caller then uses the other grouped product.
int stride_grouped_gemm_tc5(const void* A, int lda, const void* W, const int32_t* offsets, int experts, void* C, int ldc, int max_rows, int N,
                            int K, int act, float limit, float alpha, int out_is_f32, int* status, cudaStream_t stream) {
    if (max_rows < 0 || experts <= 0 || N <= 0 || K <= 0 || lda < K || act < 0 || act > 3 || ldc < (act >= 2 ? N / 2 : N) || (act >= 2 && N % 2))
        return STRIDE_BAD_ARGUMENT;
    if (status == nullptr) return STRIDE_BAD_ARGUMENT;
    if (max_rows == 0) return 0;
    if (K % 8 || lda % 8 || (reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) % 16) return STRIDE_UNSUPPORTED;
    if (static_cast<long long>(experts) * N > 2147483647LL) return STRIDE_UNSUPPORTED;
    const CUtensorMap* map_a = tc::cached_map(A, max_rows, K, lda, tc::kGroupM);
    const CUtensorMap* map_w = tc::cached_map(W, static_cast<long long>(experts) * N, K, K, 128);
    if (!map_a || !map_w) return STRIDE_UNSUPPORTED;
    // rows of four outputs are stored whole when every row of C starts on a 16-byte boundary
    const int elem = out_is_f32 ? 4 : 2;
    const int vec_ok = (reinterpret_cast<uintptr_t>(C) % 16 == 0 && (static_cast<long long>(ldc) * elem) % 16 == 0) ? 1 : 0;
    if (out_is_f32)
        return tc::launch_grouped<float>(map_a, map_w, offsets, experts, static_cast<float*>(C), ldc, max_rows, N, K, act, limit, alpha, vec_ok,
                                         status, stream);
    return tc::launch_grouped<__nv_bfloat16>(map_a, map_w, offsets, experts, static_cast<__nv_bfloat16*>(C), ldc, max_rows, N, K, act, limit,
                                             alpha, vec_ok, status, stream);
}

// xs[p] = x[perm[p]] for the rows p that the plan filled; rows of `row_bytes` (a multiple of 16), x with row stride ldx_bytes.
int stride_gather_rows(const void* x, long long ldx_bytes, const int32_t* perm, const int32_t* offsets, int experts, void* xs,
                       long long row_bytes, int max_rows, cudaStream_t stream) {
    if (max_rows < 0 || experts <= 0 || row_bytes <= 0 || ldx_bytes < row_bytes) return STRIDE_BAD_ARGUMENT;
    if (max_rows == 0) return 0;
    if (row_bytes % 16 || ldx_bytes % 16 || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(xs)) % 16) return STRIDE_UNSUPPORTED;
    const int blocks = max_rows < 148 * 8 ? max_rows : 148 * 8;
    stride::launch(tc::gather_rows_kernel, dim3(blocks), dim3(256), 0, stream, static_cast<const uint4*>(x), static_cast<int>(ldx_bytes / 16), perm,
                   offsets, experts, static_cast<uint4*>(xs), static_cast<int>(row_bytes / 16), max_rows);
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
