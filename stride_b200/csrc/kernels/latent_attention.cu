// Attention over a compressed cache: per token one latent vector c [rank] (RMS-normed) and one rotated key part
// k_r [rot] shared by all heads. Per head a the key is [W_uk_a c | k_r] and the value W_uv_a c, so with the query's
// plain part folded through W_uk (q~_a = W_uk_a^T q_a [rank]) the score of a key is
//   s = (q~_a . c + q_rot_a . k_r) * scale
// and the head's output W_uv_a (sum_j p_j c_j): every head reads the same [rank + rot] numbers per key and nothing
// but c and k_r is ever kept or expanded. Three kernels:
//
//   latent_prepare    norms the latent (float32 statistics, plain weight), rotates the shared key part and the
//                     rotated part of every query head (pairs (2i, 2i+1), angle from a float32 table), writes the
//                     latent and the key part into their pages and the rotated queries beside the folded ones;
//   head_gemm         the per-head products with W_uk (folding) and W_uv (unfolding, with an optional sigmoid gate
//                     per (token, head) in its epilogue): float32 FMA with a fixed k order for float32 operands,
//                     tensor-core tiles (mma_tile.cuh) for bfloat16;
//   latent_attention  the exact kernel: one warp per (token, head), keys walked in groups of 32 aligned to
//                     position 0 with an online softmax, so a token's result does not depend on how the step was
//                     cut; float32 arithmetic in both storage types. (The bfloat16 kernel on the tensor cores is
//                     latent_attention_tc.cu.)
#include "common.cuh"
#include "mma_tile.cuh"

namespace stride {

// ------------------------------------------------------------------------------------------------ prepare
// q: [tokens, ldq], head a at column a * (dim + rot), plain part first (a column block of proj, or a buffer of its own
// when the queries come through a latent); proj: [tokens, ld] with the latent projection (rank + rot columns) at
// kv_off, or kv_off < 0 for a layer that reads another layer's cache.
// qa: [tokens, heads, rank + rot]; this kernel fills the last rot columns of every head.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ proj, int ld, int kv_off, T* __restrict__ qa,
                      const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_of_token,
                      const int32_t* __restrict__ slot_mapping, const float* __restrict__ cos_table,
                      const float* __restrict__ sin_table, const float* __restrict__ latent_w, float eps,
                      T* __restrict__ latent_pages, T* __restrict__ krot_pages, int heads, int dim, int rot, int rot_dims, int rank) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    if (seq_of_token[t] < 0) return;
    const T* row = proj + static_cast<size_t>(t) * ld;
    const int half = rot_dims / 2;
    const float* cs = cos_table + static_cast<size_t>(positions[t]) * half;
    const float* sn = sin_table + static_cast<size_t>(positions[t]) * half;
    // rotated part of the queries
    T* qrow = qa + static_cast<size_t>(t) * heads * (rank + rot);
    for (int i = threadIdx.x; i < heads * rot; i += blockDim.x) {
        const int a = i / rot, j = i % rot;
        const T* src = q + static_cast<size_t>(t) * ldq + a * (dim + rot) + dim;
        float v = to_f32(src[j]);
        if (j < rot_dims) {
            const int pair = j >> 1;
            const float other = to_f32(src[j ^ 1]);
            v = (j & 1) ? fmaf(v, cs[pair], other * sn[pair]) : fmaf(v, cs[pair], -other * sn[pair]);
        }
        qrow[a * (rank + rot) + rank + j] = from_f32<T>(v);
    }
    if (kv_off < 0) return;
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    const T* kv = row + kv_off;
    float sq = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float x = to_f32(kv[i]);
        sq = fmaf(x, x, sq);
    }
    const float total = block_sum(sq, scratch);
    if (slot < 0) return;
    const float inv = rsqrtf(total / static_cast<float>(rank) + eps);
    T* lat = latent_pages + static_cast<size_t>(slot) * rank;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) lat[i] = from_f32<T>(to_f32(kv[i]) * inv * latent_w[i]);
    T* kr = krot_pages + static_cast<size_t>(slot) * rot;
    for (int j = threadIdx.x; j < rot; j += blockDim.x) {
        float v = to_f32(kv[rank + j]);
        if (j < rot_dims) {
            const int pair = j >> 1;
            const float other = to_f32(kv[rank + (j ^ 1)]);
            v = (j & 1) ? fmaf(v, cs[pair], other * sn[pair]) : fmaf(v, cs[pair], -other * sn[pair]);
        }
        kr[j] = from_f32<T>(v);
    }
}

// ---------------------------------------------------------------------------------------------- head_gemm
// C[t, a, n] = (sum_k A[t * lda + a * a_hs + k] * B[a * b_hs + k * b_ks + n * b_ns]) * (gate ? sigmoid(gate[t * ldg + a * g_hs + n * g_ns]) : 1)
// (g_hs 1 and g_ns 0: one gate a head; g_hs N and g_ns 1: one gate an output)
constexpr int HM = 32, HN = 64, HK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
head_gemm_kernel(const T* __restrict__ A, int lda, int a_hs, const T* __restrict__ B, long long b_hs, int b_ks, int b_ns,
                 T* __restrict__ C, int ldc, int c_hs, const T* __restrict__ gate, int ldg, int g_hs, int g_ns, int M, int N, int K) {
    pdl_trigger();
    pdl_wait();
    __shared__ float As[HK][HM + 1];
    __shared__ float Bs[HK][HN + 4];
    const int a = blockIdx.y;
    const int m0 = blockIdx.z * HM, n0 = blockIdx.x * HN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // thread: rows ty*2..+1, columns tx*4..+3
    const T* Ah = A + static_cast<size_t>(a) * a_hs;
    const T* Bh = B + static_cast<size_t>(a) * b_hs;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += HK) {
        for (int i = threadIdx.x; i < HM * HK; i += 256) {
            const int m = i / HK, k = i % HK;
            As[k][m] = (m0 + m < M && k0 + k < K) ? to_f32(Ah[static_cast<size_t>(m0 + m) * lda + k0 + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < HN * HK; i += 256) {
            int n, k;
            if (b_ns == 1) { k = i / HN; n = i % HN; } else { n = i / HK; k = i % HK; }
            Bs[k][n] = (n0 + n < N && k0 + k < K)
                           ? to_f32(Bh[static_cast<size_t>(k0 + k) * b_ks + static_cast<size_t>(n0 + n) * b_ns]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HK; ++k) {
            const float a0 = As[k][ty * 2], a1 = As[k][ty * 2 + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = Bs[k][tx * 4 + j];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = m0 + ty * 2 + i;
        if (m >= M) continue;
        float g = 1.f;
        if (gate && !g_ns) g = 1.f / (1.f + expf(-to_f32(gate[static_cast<size_t>(m) * ldg + static_cast<size_t>(a) * g_hs])));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (gate && g_ns) g = 1.f / (1.f + expf(-to_f32(gate[static_cast<size_t>(m) * ldg + static_cast<size_t>(a) * g_hs + static_cast<size_t>(n) * g_ns])));
            C[static_cast<size_t>(m) * ldc + static_cast<size_t>(a) * c_hs + n] = from_f32<T>(acc[i][j] * g);
        }
    }
}

// The same on the tensor cores for bfloat16 (mma_tile.cuh): 64 tokens x 64 columns of one head a CTA.
__global__ void __launch_bounds__(128)
head_gemm_tc_kernel(const __nv_bfloat16* __restrict__ A, int lda, int a_hs, const __nv_bfloat16* __restrict__ B, long long b_hs, int b_ks,
                    int b_ns, __nv_bfloat16* __restrict__ C, int ldc, int c_hs, const __nv_bfloat16* __restrict__ gate, int ldg, int g_hs,
                    int g_ns, int M, int N, int K) {
    pdl_trigger();
    pdl_wait();
    __shared__ TileSmem sm;
    const int a = blockIdx.y;
    const int m0 = blockIdx.z * TM, n0 = blockIdx.x * TN;
    for (int r = threadIdx.x; r < TM; r += 128)
        sm.a_rows[r] = m0 + r < M ? A + static_cast<size_t>(m0 + r) * lda + static_cast<size_t>(a) * a_hs : nullptr;
    __syncthreads();
    float acc[2][4][4];
    mma_tile_64x64(sm, B + static_cast<size_t>(a) * b_hs, b_ns, b_ks, n0, N, K, acc);
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int x = 0; x < 4; x += 2) {
            const int m = m0 + tile_row(i, x);
            if (m >= M) continue;
            float g = 1.f;
            if (gate && !g_ns) g = 1.f / (1.f + expf(-to_f32(gate[static_cast<size_t>(m) * ldg + static_cast<size_t>(a) * g_hs])));
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int y = 0; y < 2; ++y) {
                    const int n = n0 + tile_col(j, x + y);
                    if (n >= N) continue;
                    if (gate && g_ns) g = 1.f / (1.f + expf(-to_f32(gate[static_cast<size_t>(m) * ldg + static_cast<size_t>(a) * g_hs + static_cast<size_t>(n) * g_ns])));
                    C[static_cast<size_t>(m) * ldc + static_cast<size_t>(a) * c_hs + n] = __float2bfloat16_rn(acc[i][j][x + y] * g);
                }
        }
}

// ------------------------------------------------------------------------------------------- exact attention
constexpr int kLatWarps = 4;
constexpr int kMaxRank = 512;          // latent width the exact kernel keeps in registers (rank / 32 per lane)

template <typename T>
__device__ __forceinline__ float dot_span(const float* __restrict__ q, const T* __restrict__ k, int n) {
    float acc = 0.f;
    int d = 0;
    if (sizeof(T) == 2) {
        if ((reinterpret_cast<uintptr_t>(k) & 15) == 0) {
            for (; d + 8 <= n; d += 8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
                const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(pairs[i]);
                    acc = fmaf(q[d + 2 * i], f.x, acc);
                    acc = fmaf(q[d + 2 * i + 1], f.y, acc);
                }
            }
        }
    } else {
        if ((reinterpret_cast<uintptr_t>(k) & 15) == 0) {
            for (; d + 4 <= n; d += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(k + d);
                acc = fmaf(q[d], kv.x, acc);
                acc = fmaf(q[d + 1], kv.y, acc);
                acc = fmaf(q[d + 2], kv.z, acc);
                acc = fmaf(q[d + 3], kv.w, acc);
            }
        }
    }
    for (; d < n; ++d) acc = fmaf(q[d], to_f32(k[d]), acc);
    return acc;
}

// qa: [tokens, heads, rank + rot]; out: [tokens, heads, rank]; pages: latent [num_pages, page_size, rank], key part
// [num_pages, page_size, rot].
template <typename T>
__global__ void __launch_bounds__(kLatWarps * 32)
latent_attention_kernel(const T* __restrict__ qa, T* __restrict__ out, const T* __restrict__ latent_pages,
                        const T* __restrict__ krot_pages, const int32_t* __restrict__ block_table, int table_width,
                        const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ positions, int heads, int rank,
                        int rot, int page_size, float scale, const float* __restrict__ sinks) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float q_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * kLatWarps + warp;
    if (head >= heads) return;
    const int width = rank + rot;
    const int padded = (width + 3) & ~3;
    T* out_row = out + (static_cast<size_t>(t) * heads + head) * rank;
    const int seq = seq_of_token[t];
    if (seq < 0) {
        for (int d = lane; d < rank; d += 32) out_row[d] = from_f32<T>(0.f);
        return;
    }
    const int pos = positions[t];
    const int32_t* table = block_table + static_cast<size_t>(seq) * table_width;
    float* qs = q_smem + warp * padded;
    const T* q_row = qa + (static_cast<size_t>(t) * heads + head) * width;
    for (int d = lane; d < width; d += 32) qs[d] = to_f32(q_row[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[kMaxRank / 32];
#pragma unroll
    for (int i = 0; i < kMaxRank / 32; ++i) acc[i] = 0.f;

    for (int base = 0; base <= pos; base += 32) {
        const int key = base + lane;
        const bool ok = key <= pos;
        float s = -INFINITY;
        if (ok) {
            const size_t slot = static_cast<size_t>(table[key / page_size]) * page_size + key % page_size;
            s = (dot_span<T>(qs, latent_pages + slot * rank, rank) + dot_span<T>(qs + rank, krot_pages + slot * rot, rot)) * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = ok ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < kMaxRank / 32; ++i) acc[i] *= corr;
        const int count = min(32, pos - base + 1);
        for (int j = 0; j < count; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const int kj = base + j;
            const T* v_row = latent_pages + (static_cast<size_t>(table[kj / page_size]) * page_size + kj % page_size) * rank;
#pragma unroll
            for (int i = 0; i < kMaxRank / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < rank) acc[i] = fmaf(pj, to_f32(v_row[d]), acc[i]);
            }
        }
        m = m_new;
    }
    float inv = 1.f / l;
    if (sinks) {        // exp(sink_h) joins the denominator after the last key group: the order of the sums depends on the position only
        const float sink = sinks[head], top = fmaxf(m, sink);
        const float keep = expf(m - top);
        inv = keep / (l * keep + expf(sink - top));
    }
#pragma unroll
    for (int i = 0; i < kMaxRank / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) out_row[d] = from_f32<T>(acc[i] * inv);
    }
}

}  // namespace stride

using namespace stride;

extern "C" {

int stride_latent_prepare(const void* q, int ldq, const void* proj, int ld, int kv_off, void* qa, const int32_t* positions,
                          const int32_t* seq_of_token, const int32_t* slot_mapping, const float* cos_table, const float* sin_table,
                          const float* latent_w, float eps, void* latent_pages, void* krot_pages, int tokens, int heads, int dim,
                          int rot, int rot_dims, int rank, int dtype, cudaStream_t stream) {
    if (tokens < 0 || heads <= 0 || dim <= 0 || rot < 0 || rank <= 0 || rot_dims < 0 || rot_dims > rot || rot_dims % 2 || ld <= 0 || ldq <= 0 || !q)
        return STRIDE_BAD_ARGUMENT;
    if (kv_off >= 0 && (!latent_w || !latent_pages || (rot > 0 && !krot_pages))) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(latent_prepare_kernel<float>, dim3(tokens), dim3(128), 0, stream, static_cast<const float*>(q), ldq,
                       static_cast<const float*>(proj), ld, kv_off,
                       static_cast<float*>(qa), positions, seq_of_token, slot_mapping, cos_table, sin_table, latent_w, eps,
                       static_cast<float*>(latent_pages), static_cast<float*>(krot_pages), heads, dim, rot, rot_dims, rank);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(latent_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(q), ldq,
                       static_cast<const __nv_bfloat16*>(proj), ld, kv_off, static_cast<__nv_bfloat16*>(qa), positions, seq_of_token, slot_mapping, cos_table, sin_table,
                       latent_w, eps, static_cast<__nv_bfloat16*>(latent_pages), static_cast<__nv_bfloat16*>(krot_pages), heads, dim,
                       rot, rot_dims, rank);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_head_gemm(const void* A, int lda, int a_hs, const void* B, long long b_hs, int b_ks, int b_ns, void* C, int ldc, int c_hs,
                     const void* gate, int ldg, int g_hs, int g_ns, int M, int heads, int N, int K, int dtype, cudaStream_t stream) {
    if (M < 0 || heads <= 0 || N <= 0 || K <= 0 || heads > 65535 || g_hs < 0 || g_ns < 0) return STRIDE_BAD_ARGUMENT;
    if (M == 0) return 0;
    const dim3 grid((N + HN - 1) / HN, heads, (M + HM - 1) / HM);
    if (grid.z > 65535) return STRIDE_UNSUPPORTED;
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(head_gemm_kernel<float>, grid, dim3(256), 0, stream, static_cast<const float*>(A), lda, a_hs,
                       static_cast<const float*>(B), b_hs, b_ks, b_ns, static_cast<float*>(C), ldc, c_hs, static_cast<const float*>(gate),
                       ldg, g_hs, g_ns, M, N, K);
    else if (dtype == STRIDE_DTYPE_BF16) {
        const dim3 tc_grid((N + TN - 1) / TN, heads, (M + TM - 1) / TM);
        stride::launch(head_gemm_tc_kernel, tc_grid, dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(A), lda, a_hs,
                       static_cast<const __nv_bfloat16*>(B), b_hs, b_ks, b_ns, static_cast<__nv_bfloat16*>(C), ldc, c_hs,
                       static_cast<const __nv_bfloat16*>(gate), ldg, g_hs, g_ns, M, N, K);
    }
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_latent_attention(const void* qa, void* out, const void* latent_pages, const void* krot_pages, const int32_t* block_table,
                            int table_width, const int32_t* seq_of_token, const int32_t* positions, int tokens, int heads, int rank,
                            int rot, int page_size, float scale, const float* sinks, int dtype, cudaStream_t stream) {
    if (tokens < 0 || heads <= 0 || rank <= 0 || rot < 0 || page_size <= 0 || table_width <= 0) return STRIDE_BAD_ARGUMENT;
    if (rank > kMaxRank) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    const size_t smem = static_cast<size_t>(kLatWarps) * ((rank + rot + 3) & ~3) * sizeof(float);
    if (smem > 48 * 1024) return STRIDE_UNSUPPORTED;
    const dim3 grid(tokens, (heads + kLatWarps - 1) / kLatWarps);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(latent_attention_kernel<float>, grid, dim3(kLatWarps * 32), smem, stream, static_cast<const float*>(qa),
                       static_cast<float*>(out), static_cast<const float*>(latent_pages), static_cast<const float*>(krot_pages), block_table,
                       table_width, seq_of_token, positions, heads, rank, rot, page_size, scale, sinks);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(latent_attention_kernel<__nv_bfloat16>, grid, dim3(kLatWarps * 32), smem, stream,
                       static_cast<const __nv_bfloat16*>(qa), static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(latent_pages),
                       static_cast<const __nv_bfloat16*>(krot_pages), block_table, table_width, seq_of_token, positions, heads, rank, rot,
                       page_size, scale, sinks);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
