// Latent attention on the tensor cores (bfloat16, mma.sync m16n8k16, float32 accumulators), for portions of prompts
// and for single decoded tokens.
//
// Every head of a token reads the same keys ([latent | rotated part], rank + rot numbers a key) and the same values
// (the latent), so the rows of the M tile are (token, head) pairs of one request: one tile of keys in shared memory
// serves heads x tokens rows, as many-query attention with one key head. A CTA owns ROWS = 16 * MT rows and walks the
// keys in tiles of 64:
//
//   S = Q K^T      each warp a slice of the 64 keys, all rows; K dimension rank + rot
//   softmax        running maximum and sum per row, exchanged between the warps through shared memory
//   O += P V       each warp a slice of the rank columns, all rows; P in bfloat16 from shared memory; V is the latent
//                  part of the same key tile, read as the transposed operand with ldmatrix
//
// MT = 4 with 8 warps serves portions (64 rows = 64 / heads tokens), MT = 1 with 4 warps single tokens, where the keys
// may be split over CTAs: a split leaves (max, sum, unnormalised O) per row in scratch and a second kernel merges them in
// the order of the splits. A row's keys end at its token's position; the result of a row depends on its own keys only.
// An optional sink per head (`sinks`, float32 [heads]) adds exp(sink) to a row's denominator, after the last key (in the
// merge when the keys are split).
// Sizes: rank and rot multiples of 16, rank <= 512, rank + rot <= 640.
#include "common.cuh"

namespace stride {

constexpr int KT = 64;                 // keys a tile
constexpr int kTcMaxRank = 512;

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* smem_row) {
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, const void* smem_row) {
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}

// 16 bytes from global to shared memory without a register in between; `bytes` 0 writes zeros. Many of them are in
// flight per thread, which is what makes a tile of scattered rows arrive in one memory latency and not in one a row.
__device__ __forceinline__ void copy16_async(void* smem_dst, const void* src, int bytes) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copies_done() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// qa: [tokens, heads, rank + rot]; out: [tokens, heads, rank]; partial: [tokens * heads, splits, rank + 2] float32
// (max, sum, O) when splits > 1. Grid: (row tiles of the longest request, requests, splits).
template <int MT, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
latent_attention_tc_kernel(const __nv_bfloat16* __restrict__ qa, __nv_bfloat16* __restrict__ out, float* __restrict__ partial,
                           const __nv_bfloat16* __restrict__ latent_pages, const __nv_bfloat16* __restrict__ krot_pages,
                           const int32_t* __restrict__ block_table, int table_width, const int32_t* __restrict__ q_start,
                           const int32_t* __restrict__ q_len, const int32_t* __restrict__ ctx_len, int first_seq, int heads, int rank,
                           int rot, int page_size, float scale, int splits, int keys_per_split, const float* __restrict__ sinks) {
    constexpr int ROWS = MT * 16;
    constexpr int KW = KT / NW;                    // keys a warp scores
    constexpr int SN = KW / 8;                     // n8 tiles of S a warp
    constexpr int MAXT = kTcMaxRank / 8 / NW;      // n8 tiles of O a warp, at most
    pdl_trigger();
    pdl_wait();
    const int seq = first_seq + blockIdx.y;
    const int n = q_len[seq];
    if (n <= 0) return;
    const int total_rows = n * heads;
    const int r0 = blockIdx.x * ROWS;
    if (r0 >= total_rows) return;
    const int split = blockIdx.z;
    const int start = q_start[seq];
    const int pos0 = ctx_len[seq] - n;             // position of the request's first token in this step
    const int width = rank + rot, ld = width + 8;
    const int last_row = min(total_rows, r0 + ROWS) - 1;
    const int k_limit = pos0 + last_row / heads + 1;                    // keys any row of the tile may read
    const int k_begin = split * keys_per_split;
    const int k_end = min(k_limit, k_begin + keys_per_split);

    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                  // [ROWS][ld]
    __nv_bfloat16* Ks = Qs + ROWS * ld;                                               // [KT][ld]
    __nv_bfloat16* Ps = Ks + KT * ld;                                                 // [ROWS][KT + 8]
    float* red_max = reinterpret_cast<float*>(Ps + ROWS * (KT + 8));                  // [NW][ROWS]
    float* red_sum = red_max + NW * ROWS;                                             // [NW][ROWS]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int chunks = width / 8;
    const size_t first_global_row = static_cast<size_t>(start) * heads + r0;
    for (int c = tid; c < ROWS * chunks; c += NW * 32) {
        const int r = c / chunks, x = (c % chunks) * 8;
        const bool live = r0 + r < total_rows;
        copy16_async(Qs + r * ld + x, qa + (first_global_row + (live ? r : 0)) * width + x, live ? 16 : 0);
    }
    const int32_t* table = block_table + static_cast<size_t>(seq) * table_width;
    const int ntiles = rank / 8;

    float acc_o[MT][MAXT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < MAXT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc_o[i][j][e] = 0.f;
    float m_run[MT][2], l_run[MT][2];
    int row_pos[MT][2];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            m_run[i][h] = -INFINITY;
            l_run[i][h] = 0.f;
            const int row = r0 + i * 16 + g + 8 * h;
            row_pos[i][h] = row < total_rows ? pos0 + row / heads : -1;        // -1: no key is visible
        }

    for (int kt = k_begin; kt < k_end; kt += KT) {
        // ---- the key tile: [latent | rotated part] of 64 keys through the block table
        for (int c = tid; c < KT * chunks; c += NW * 32) {
            const int j = c / chunks, x = (c % chunks) * 8;
            const int key = min(kt + j, k_end - 1);                 // a key beyond the end: zeros, whatever the address
            const size_t slot = static_cast<size_t>(table[key / page_size]) * page_size + key % page_size;
            const __nv_bfloat16* src = x < rank ? latent_pages + slot * rank + x : krot_pages + slot * rot + (x - rank);
            copy16_async(Ks + j * ld + x, src, kt + j < k_end ? 16 : 0);
        }
        copies_done();
        __syncthreads();
        // ---- S = Q K^T for this warp's keys
        float acc_s[MT][SN][4];
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < SN; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc_s[i][j][e] = 0.f;
        for (int kk = 0; kk < width; kk += 16) {
            // fragments by ldmatrix: a key tile's rows are keys with the K dimension along them, which is the layout of
            // the B operand as it stands (matrices: keys 0-7 x k 0-7, keys 0-7 x k 8-15)
            uint32_t bf[SN][2];
#pragma unroll
            for (int j = 0; j < SN; ++j)
                ldmatrix_x2(bf[j][0], bf[j][1], Ks + (warp * KW + j * 8 + (lane & 7)) * ld + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                uint32_t af[4];
                ldmatrix_x4(af, Qs + (i * 16 + (lane & 15)) * ld + kk + (lane >> 4) * 8);
#pragma unroll
                for (int j = 0; j < SN; ++j) mma16816(acc_s[i][j], af, bf[j][0], bf[j][1]);
            }
        }
        // ---- mask, this warp's maximum per row
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < SN; ++j)
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        const int key = kt + warp * KW + j * 8 + 2 * t + b;
                        const bool ok = key <= row_pos[i][h] && key < k_end;
                        const float s = ok ? acc_s[i][j][2 * h + b] * scale : -INFINITY;
                        acc_s[i][j][2 * h + b] = s;
                        mx = fmaxf(mx, s);
                    }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                if (t == 0) red_max[warp * ROWS + i * 16 + g + 8 * h] = mx;
            }
        __syncthreads();
        float corr[MT][2];
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = i * 16 + g + 8 * h;
                float m_new = m_run[i][h];
#pragma unroll
                for (int w = 0; w < NW; ++w) m_new = fmaxf(m_new, red_max[w * ROWS + row]);
                corr[i][h] = m_new == -INFINITY ? 1.f : expf(m_run[i][h] - m_new);
                m_run[i][h] = m_new;
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < SN; ++j) {
                    const float s0 = acc_s[i][j][2 * h], s1 = acc_s[i][j][2 * h + 1];
                    const float p0 = s0 == -INFINITY ? 0.f : expf(s0 - m_new), p1 = s1 == -INFINITY ? 0.f : expf(s1 - m_new);
                    const __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
                    sum += __bfloat162float(pr.x) + __bfloat162float(pr.y);       // the sum of what the second product uses
                    *reinterpret_cast<__nv_bfloat162*>(Ps + row * (KT + 8) + warp * KW + j * 8 + 2 * t) = pr;
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if (t == 0) red_sum[warp * ROWS + row] = sum;
            }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = i * 16 + g + 8 * h;
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < NW; ++w) sum += red_sum[w * ROWS + row];
                l_run[i][h] = l_run[i][h] * corr[i][h] + sum;
#pragma unroll
                for (int j = 0; j < MAXT; ++j) {
                    acc_o[i][j][2 * h] *= corr[i][h];
                    acc_o[i][j][2 * h + 1] *= corr[i][h];
                }
            }
        // ---- O += P V for this warp's columns of the latent
#pragma unroll
        for (int ks = 0; ks < KT; ks += 16) {
            uint32_t af[MT][4];
#pragma unroll
            for (int i = 0; i < MT; ++i) ldmatrix_x4(af[i], Ps + (i * 16 + (lane & 15)) * (KT + 8) + ks + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < MAXT; ++j) {
                const int tile = warp + j * NW;
                if (tile < ntiles) {
                    uint32_t b0, b1;
                    ldmatrix_x2_trans(b0, b1, Ks + (ks + (lane & 15)) * ld + tile * 8);
#pragma unroll
                    for (int i = 0; i < MT; ++i) mma16816(acc_o[i][j], af[i], b0, b1);
                }
            }
        }
        __syncthreads();
    }

    copies_done();          // a CTA without keys still has its queries on the way
    // ---- result
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = r0 + i * 16 + g + 8 * h;
            if (row >= total_rows) continue;
            const size_t grow = static_cast<size_t>(start) * heads + row;
            if (splits == 1) {
                float inv = 1.f / l_run[i][h];
                if (sinks) {            // exp(sink) joins the sum; both terms relative to the larger of the maximum and the sink
                    const float sink = sinks[row % heads], top = fmaxf(m_run[i][h], sink);
                    const float keep = expf(m_run[i][h] - top);
                    inv = keep / (l_run[i][h] * keep + expf(sink - top));
                }
#pragma unroll
                for (int j = 0; j < MAXT; ++j) {
                    const int tile = warp + j * NW;
                    if (tile < ntiles)
                        *reinterpret_cast<uint32_t*>(out + grow * rank + tile * 8 + 2 * t) =
                            pack_bf16(acc_o[i][j][2 * h] * inv, acc_o[i][j][2 * h + 1] * inv);
                }
            } else {
                float* dst = partial + (grow * splits + split) * (rank + 2);
                if (warp == 0 && t == 0) {
                    dst[0] = m_run[i][h];
                    dst[1] = l_run[i][h];
                }
#pragma unroll
                for (int j = 0; j < MAXT; ++j) {
                    const int tile = warp + j * NW;
                    if (tile < ntiles) {
                        dst[2 + tile * 8 + 2 * t] = acc_o[i][j][2 * h];
                        dst[2 + tile * 8 + 2 * t + 1] = acc_o[i][j][2 * h + 1];
                    }
                }
            }
        }
}

// One warp per (token, head): the splits' partial results, combined in the order of the splits. Every lane first takes
// the weight exp(m_s - m) / L of the splits s = lane and lane + 32 (at most 64 splits), so that the sums over the latent's
// columns are independent loads and multiply-adds.
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ seq_of_token,
                    int first_token, int rows, int heads, int rank, int splits, const float* __restrict__ sinks) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= rows) return;
    const size_t grow = static_cast<size_t>(first_token) * heads + r;
    if (seq_of_token[first_token + r / heads] < 0) return;
    const size_t stride = static_cast<size_t>(rank) + 2;
    const float* src = partial + grow * splits * stride;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    if (lane < splits) { m0 = src[lane * stride]; l0 = src[lane * stride + 1]; }
    if (lane + 32 < splits) { m1 = src[(lane + 32) * stride]; l1 = src[(lane + 32) * stride + 1]; }
    const float m = warp_max(fmaxf(m0, m1));
    float w0 = m0 == -INFINITY ? 0.f : expf(m0 - m), w1 = m1 == -INFINITY ? 0.f : expf(m1 - m);
    // the sum of the splits' sums in the order of the splits
    float l = 0.f;
    for (int s2 = 0; s2 < splits; ++s2) {
        const float ws = __shfl_sync(0xffffffffu, s2 < 32 ? w0 : w1, s2 & 31), ls = __shfl_sync(0xffffffffu, s2 < 32 ? l0 : l1, s2 & 31);
        l = fmaf(ls, ws, l);
    }
    float inv = 1.f / l;
    if (sinks) {
        const float sink = sinks[r % heads], top = fmaxf(m, sink);
        const float keep = expf(m - top);
        inv = keep / (l * keep + expf(sink - top));
    }
    w0 *= inv;
    w1 *= inv;
    for (int d = lane; d < rank; d += 32) {
        float acc = 0.f;
#pragma unroll 4
        for (int s2 = 0; s2 < splits; ++s2) {
            const float ws = __shfl_sync(0xffffffffu, s2 < 32 ? w0 : w1, s2 & 31);
            acc = fmaf(src[s2 * stride + 2 + d], ws, acc);
        }
        out[grow * rank + d] = __float2bfloat16_rn(acc);
    }
}

template <int MT, int NW>
static size_t tc_smem_bytes(int rank, int rot) {
    const int ld = rank + rot + 8;
    return static_cast<size_t>(MT * 16 + KT) * ld * 2 + static_cast<size_t>(MT * 16) * (KT + 8) * 2 + 2ull * NW * MT * 16 * 4;
}

}  // namespace stride

using namespace stride;

extern "C" {

// Keys a split takes for single tokens at this context bound, a multiple of the key tile; 0: the sizes are not taken.
int stride_latent_tc_supported(int heads, int rank, int rot) {
    return rank > 0 && rot >= 0 && rank % 16 == 0 && rot % 16 == 0 && rank <= kTcMaxRank && rank + rot <= 640 && heads > 0;
}

// The requests first_seq .. first_seq + num_seqs - 1 of the step, which own the rows first_token .. of qa and out.
// max_rows: heads * the most tokens one of them brings. splits > 1 needs `partial` of tokens * heads * splits * (rank + 2)
// floats and runs the merge.
int stride_latent_attention_tc(const void* qa, void* out, float* partial, const void* latent_pages, const void* krot_pages,
                               const int32_t* block_table, int table_width, const int32_t* q_start, const int32_t* q_len,
                               const int32_t* ctx_len, const int32_t* seq_of_token, int first_seq, int num_seqs, int first_token,
                               int tokens, int max_q_len, int heads, int rank, int rot, int page_size, float scale, int splits,
                               int keys_per_split, const float* sinks, cudaStream_t stream) {
    if (num_seqs < 0 || tokens < 0 || max_q_len <= 0 || page_size <= 0 || table_width <= 0 || splits <= 0) return STRIDE_BAD_ARGUMENT;
    if (!stride_latent_tc_supported(heads, rank, rot)) return STRIDE_UNSUPPORTED;
    if (splits > 1 && (!partial || keys_per_split <= 0 || keys_per_split % KT)) return STRIDE_BAD_ARGUMENT;
    if (num_seqs == 0 || tokens == 0) return 0;
    if (num_seqs > 65535 || splits > 64) return STRIDE_UNSUPPORTED;
    const int kps = splits > 1 ? keys_per_split : 0x3fffffc0;
    const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(qa);
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
    const __nv_bfloat16* lp = static_cast<const __nv_bfloat16*>(latent_pages);
    const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(krot_pages);
    const long long max_rows = static_cast<long long>(max_q_len) * heads;
    if (max_q_len == 1) {
        auto kernel = latent_attention_tc_kernel<1, 4>;
        const size_t smem = tc_smem_bytes<1, 4>(rank, rot);
        static size_t set = 0;
        if (smem > set) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
                return STRIDE_UNSUPPORTED;
            set = smem;
        }
        const dim3 grid(static_cast<unsigned>((max_rows + 15) / 16), num_seqs, splits);
        stride::launch(kernel, grid, dim3(128), smem, stream, q, o, partial, lp, kp, block_table, table_width, q_start, q_len, ctx_len,
                       first_seq, heads, rank, rot, page_size, scale, splits, kps, splits == 1 ? sinks : nullptr);
    } else {
        if (splits != 1) return STRIDE_BAD_ARGUMENT;
        auto kernel = latent_attention_tc_kernel<4, 8>;
        const size_t smem = tc_smem_bytes<4, 8>(rank, rot);
        static size_t set = 0;
        if (smem > set) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
                return STRIDE_UNSUPPORTED;
            set = smem;
        }
        const dim3 grid(static_cast<unsigned>((max_rows + 63) / 64), num_seqs, 1);
        stride::launch(kernel, grid, dim3(256), smem, stream, q, o, partial, lp, kp, block_table, table_width, q_start, q_len, ctx_len,
                       first_seq, heads, rank, rot, page_size, scale, 1, kps, sinks);
    }
    int status = STRIDE_LAUNCH_STATUS();
    if (status != 0 || splits == 1) return status;
    const int rows = tokens * heads;
    stride::launch(latent_merge_kernel, dim3((rows + 3) / 4), dim3(128), 0, stream, static_cast<const float*>(partial), o, seq_of_token,
                   first_token, rows, heads, rank, splits, sinks);
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
