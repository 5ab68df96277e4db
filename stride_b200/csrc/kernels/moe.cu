// Routed feed-forward: each token goes to the `top` experts with the largest router logits.
//
//   moe_route     router logits z = W_r h + b in float32 (one warp per token), the top entries (the lower index wins
//                 among equals), and the softmax over the chosen logits only; moe_select is the choice alone, from
//                 logits that a matrix product with float32 output has made (what the part runs);
//   moe_select_sigmoid  the choice by another rule: scores s = sigmoid(z); choice scores c = s + correction; the experts form
//                 equal groups of neighbours, a group's score is the sum of its two largest c, only the experts of the
//                 `keep` best groups can be chosen (the others count as minus infinity); the `top` largest c win (the
//                 lower index among equals); weights s / (sum of the chosen s + 1e-20) * route_scale. `rule` bits change
//                 it: 1 makes s the softmax of z over all experts, 2 makes a group's score its largest c, 4 leaves the
//                 weights at s * route_scale (no division by their sum);
//   moe_plan      one CTA counts the rows of every expert, lays the (token, choice) pairs out expert by expert and
//                 writes where each pair went: `offsets` [experts + 1], `perm_token` [rows] and `row_of` [tokens, top];
//   grouped_gemm  C[p, :] = act(A[src(p), :] W[e(p)]^T) for the rows p of every expert e, the tiles of all experts in
//                 one launch (the CTA finds its expert from `offsets` on the device, so nothing goes back to the
//                 host and the step can be replayed from a graph); float32 FMA with a fixed k order for float32
//                 operands, tensor-core tiles (mma_tile.cuh) for bfloat16;
//                 act 1 squares the positive part; act 2 reads W's rows as (gate, up) pairs, row 2i beside row 2i + 1,
//                 and writes g' sigmoid(alpha g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit), N / 2 wide;
//                 act 3 reads the same pairs and writes g sigmoid(g) u;
//   moe_combine   out[t] = sum_k weight[t, k] * Y[row_of[t, k]] (+ a shared expert's output, optionally times the
//                 sigmoid of a per-token logit), in the order of k.
// A row's result depends only on that row: not on the batch, nor on where the plan put it.
#include "common.cuh"
#include "mma_tile.cuh"

namespace stride {

constexpr int kMaxExperts = 256;
constexpr int kMaxTop = 32;
constexpr int kRuleSoftmax = 1, kRuleGroupMax = 2, kRuleKeepScores = 4;      // bits of the group router's `rule`

template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ h, const T* __restrict__ w_router, const float* __restrict__ bias,
                 const int32_t* __restrict__ seq_of_token, int32_t* __restrict__ ids, float* __restrict__ weights, int tokens,
                 int hidden, int experts, int top) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= tokens) return;
    if (seq_of_token && seq_of_token[t] < 0) {
        for (int k = lane; k < top; k += 32) {
            ids[static_cast<size_t>(t) * top + k] = -1;
            weights[static_cast<size_t>(t) * top + k] = 0.f;
        }
        return;
    }
    const T* x = h + static_cast<size_t>(t) * hidden;
    float z[kMaxExperts / 32];          // lane holds the logits of experts lane, lane + 32, ...
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) z[i] = -INFINITY;
    for (int e = 0; e < experts; ++e) {
        const T* w = w_router + static_cast<size_t>(e) * hidden;
        float acc = 0.f;
        for (int i = lane; i < hidden; i += 32) acc = fmaf(to_f32(x[i]), to_f32(w[i]), acc);
        acc = warp_sum(acc) + (bias ? bias[e] : 0.f);
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i)
            if (i == e / 32 && lane == e % 32) z[i] = acc;
    }
    float first = 0.f, denom = 0.f, mine = 0.f;
    int mine_id = -1;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i) {
            const int e = i * 32 + lane;
            if (e < experts && (z[i] > best)) { best = z[i]; best_e = e; }      // ascending e: the lower index stays on a tie
        }
        if (best == -INFINITY) best_e = 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i)
            if (i * 32 + lane == best_e) z[i] = -INFINITY;       // taken
        if (k == 0) first = best;
        const float p = expf(best - first);
        denom += p;
        if (lane == k) { mine = p; mine_id = best_e; }
    }
    if (lane < top) {
        ids[static_cast<size_t>(t) * top + lane] = mine_id;
        weights[static_cast<size_t>(t) * top + lane] = mine / denom;
    }
}

// The choice alone, from logits a matrix product has made: z = logits + bias in float32, the same top rule and softmax.
__global__ void __launch_bounds__(128)
moe_select_kernel(const float* __restrict__ logits, const float* __restrict__ bias, const int32_t* __restrict__ seq_of_token,
                  int32_t* __restrict__ ids, float* __restrict__ weights, int tokens, int experts, int top) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= tokens) return;
    if (seq_of_token && seq_of_token[t] < 0) {
        for (int k = lane; k < top; k += 32) {
            ids[static_cast<size_t>(t) * top + k] = -1;
            weights[static_cast<size_t>(t) * top + k] = 0.f;
        }
        return;
    }
    float z[kMaxExperts / 32];
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) {
        const int e = i * 32 + lane;
        z[i] = e < experts ? logits[static_cast<size_t>(t) * experts + e] + (bias ? bias[e] : 0.f) : -INFINITY;
    }
    float first = 0.f, denom = 0.f, mine = 0.f;
    int mine_id = -1;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i) {
            const int e = i * 32 + lane;
            if (e < experts && (z[i] > best)) { best = z[i]; best_e = e; }
        }
        if (best == -INFINITY) best_e = 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i)
            if (i * 32 + lane == best_e) z[i] = -INFINITY;
        if (k == 0) first = best;
        const float p = expf(best - first);
        denom += p;
        if (lane == k) { mine = p; mine_id = best_e; }
    }
    if (lane < top) {
        ids[static_cast<size_t>(t) * top + lane] = mine_id;
        weights[static_cast<size_t>(t) * top + lane] = mine / denom;
    }
}

// logits: [tokens, ld] float32 (the first `experts` columns of a row). One warp per token.
__global__ void __launch_bounds__(128)
moe_select_sigmoid_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ correction,
                          const int32_t* __restrict__ seq_of_token, int32_t* __restrict__ ids, float* __restrict__ weights, int tokens,
                          int experts, int top, int groups, int keep, float route_scale, int rule) {
    pdl_trigger();
    pdl_wait();
    __shared__ float choice_s[4][kMaxExperts];
    __shared__ float group_s[4][kMaxExperts];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= tokens) return;
    if (seq_of_token && seq_of_token[t] < 0) {
        for (int k = lane; k < top; k += 32) {
            ids[static_cast<size_t>(t) * top + k] = -1;
            weights[static_cast<size_t>(t) * top + k] = 0.f;
        }
        return;
    }
    float* choice = choice_s[warp];
    float* gscore = group_s[warp];
    float score[kMaxExperts / 32];       // lane holds experts lane, lane + 32, ...
    if (rule & kRuleSoftmax) {           // softmax over all experts: largest logit, exponentials, their sum in a fixed order
        float top_z = -INFINITY;
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i) {
            const int e = i * 32 + lane;
            score[i] = e < experts ? logits[static_cast<size_t>(t) * ld + e] : -INFINITY;
            top_z = fmaxf(top_z, score[i]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) top_z = fmaxf(top_z, __shfl_xor_sync(0xffffffffu, top_z, o));
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i) {
            score[i] = i * 32 + lane < experts ? expf(score[i] - top_z) : 0.f;
            sum += score[i];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i) {
            const int e = i * 32 + lane;
            score[i] /= sum;
            if (e < experts) choice[e] = score[i] + (correction ? correction[e] : 0.f);
        }
    } else {
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i) {
            const int e = i * 32 + lane;
            score[i] = 0.f;
            if (e < experts) {
                score[i] = 1.f / (1.f + expf(-logits[static_cast<size_t>(t) * ld + e]));
                choice[e] = score[i] + (correction ? correction[e] : 0.f);
            }
        }
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int size = experts / groups;
        for (int g = lane; g < groups; g += 32) {       // the two largest choice scores of the group
            float a = -INFINITY, b = -INFINITY;
            for (int e = g * size; e < (g + 1) * size; ++e) {
                const float c = choice[e];
                if (c > a) { b = a; a = c; }
                else if (c > b) b = c;
            }
            gscore[g] = (size > 1 && !(rule & kRuleGroupMax)) ? a + b : a;
        }
        __syncwarp();
        unsigned kept[kMaxExperts / 32] = {};           // bit l of kept[i]: group i * 32 + l stays
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY;
            int best_g = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const bool taken = (kept[g >> 5] >> (g & 31)) & 1u;
                if (!taken && (best_g == 0x7fffffff || gscore[g] > best)) { best = gscore[g]; best_g = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
                if (og != 0x7fffffff && (best_g == 0x7fffffff || ob > best || (ob == best && og < best_g))) { best = ob; best_g = og; }
            }
            if (best_g != 0x7fffffff) kept[best_g >> 5] |= 1u << (best_g & 31);        // every lane keeps the whole set
        }
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i) {
            const int e = i * 32 + lane;
            if (e < experts) {
                const int g = e / size;
                if (!((kept[g >> 5] >> (g & 31)) & 1u)) choice[e] = -INFINITY;
            }
        }
        __syncwarp();
    }
    float z[kMaxExperts / 32];
    bool open_[kMaxExperts / 32];
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) {
        const int e = i * 32 + lane;
        open_[i] = e < experts;
        z[i] = e < experts ? choice[e] : -INFINITY;
    }
    float denom = 0.f, mine = 0.f;
    int mine_id = -1;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY, best_score = 0.f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i) {
            const int e = i * 32 + lane;
            if (open_[i] && (best_e == 0x7fffffff || z[i] > best)) { best = z[i]; best_e = e; best_score = score[i]; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const float os = __shfl_xor_sync(0xffffffffu, best_score, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (oe != 0x7fffffff && (best_e == 0x7fffffff || ob > best || (ob == best && oe < best_e))) { best = ob; best_e = oe; best_score = os; }
        }
#pragma unroll
        for (int i = 0; i < kMaxExperts / 32; ++i)
            if (i * 32 + lane == best_e) open_[i] = false;       // taken
        denom += best_score;
        if (lane == k) { mine = best_score; mine_id = best_e == 0x7fffffff ? -1 : best_e; }
    }
    if (lane < top) {
        ids[static_cast<size_t>(t) * top + lane] = mine_id;
        weights[static_cast<size_t>(t) * top + lane] = (rule & kRuleKeepScores) ? mine * route_scale : mine / (denom + 1e-20f) * route_scale;
    }
}

// ids: [tokens, top] (-1: a padded token). rank_tmp: [tokens * top] scratch.
__global__ void __launch_bounds__(256)
moe_plan_kernel(const int32_t* __restrict__ ids, int pairs, int experts, int32_t* __restrict__ offsets, int32_t* __restrict__ perm_token,
                int32_t* __restrict__ row_of, int32_t* __restrict__ rank_tmp, int top) {
    pdl_trigger();
    pdl_wait();
    __shared__ int counts[kMaxExperts];
    __shared__ int starts[kMaxExperts + 1];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < experts) rank_tmp[i] = atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            starts[e] = at;
            at += counts[e];
        }
        starts[experts] = at;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = starts[e];
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < experts) {
            const int row = starts[e] + rank_tmp[i];
            row_of[i] = row;
            perm_token[row] = i / top;
        } else {
            row_of[i] = -1;
        }
    }
}

__device__ __forceinline__ float clamped_gated(float g, float u, float limit, float alpha) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}

// What a (gate, up) pair becomes: act 2 the clamped form, act 3 plain SiLU(g) * u.
__device__ __forceinline__ float gated_pair(int act, float g, float u, float limit, float alpha) {
    return act == 3 ? g / (1.f + expf(-g)) * u : clamped_gated(g, u, limit, alpha);
}

// Tiles of GM x GN outputs; tile `blockIdx.y` belongs to the expert whose tiles it falls among.
constexpr int GM = 64, GN = 64, GK = 16;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const TA* __restrict__ A, int lda, const int32_t* __restrict__ row_map, const TW* __restrict__ W,
                    const int32_t* __restrict__ offsets, int experts, TC* __restrict__ C, int ldc, int N, int K, int act, float limit,
                    float alpha) {
    pdl_trigger();
    pdl_wait();
    __shared__ float As[GK][GM + 4];
    __shared__ float Ws[GK][GN + 4];
    __shared__ int src_row[GM];
    int tile = blockIdx.y, e = 0, m0 = 0, m_end = 0;
    for (; e < experts; ++e) {
        const int lo = offsets[e], hi = offsets[e + 1];
        const int tiles = (hi - lo + GM - 1) / GM;
        if (tile < tiles) {
            m0 = lo + tile * GM;
            m_end = hi;
            break;
        }
        tile -= tiles;
    }
    if (e >= experts) return;
    const int n0 = blockIdx.x * GN;
    const TW* We = W + static_cast<size_t>(e) * N * K;
    for (int i = threadIdx.x; i < GM; i += 256) src_row[i] = m0 + i < m_end ? (row_map ? row_map[m0 + i] : m0 + i) : -1;
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int lrow = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += GK) {
        const int srow = src_row[lrow];
        const int wn = n0 + lrow;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            As[lk + j][lrow] = (srow >= 0 && k < K) ? to_f32(A[static_cast<size_t>(srow) * lda + k]) : 0.f;
            Ws[lk + j][lrow] = (wn < N && k < K) ? to_f32(We[static_cast<size_t>(wn) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= m_end) continue;
        if (act >= 2) {                     // columns come in (gate, up) pairs
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int n = n0 + tx * 4 + j;
                if (n + 1 < N) C[static_cast<size_t>(m) * ldc + n / 2] = from_f32<TC>(gated_pair(act, acc[i][j], acc[i][j + 1], limit, alpha));
            }
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (act == 1) {                 // the square of relu
                v = fmaxf(v, 0.f);
                v *= v;
            }
            C[static_cast<size_t>(m) * ldc + n] = from_f32<TC>(v);
        }
    }
}

// The same on the tensor cores for bfloat16 operands (mma_tile.cuh): 128 threads a tile.
template <typename TC>
__global__ void __launch_bounds__(128)
grouped_gemm_tc_kernel(const __nv_bfloat16* __restrict__ A, int lda, const int32_t* __restrict__ row_map,
                       const __nv_bfloat16* __restrict__ W, const int32_t* __restrict__ offsets, int experts, TC* __restrict__ C, int ldc,
                       int N, int K, int act, float limit, float alpha) {
    pdl_trigger();
    pdl_wait();
    __shared__ TileSmem sm;
    int tile = blockIdx.y, e = 0, m0 = 0, m_end = 0;
    for (; e < experts; ++e) {
        const int lo = offsets[e], hi = offsets[e + 1];
        const int tiles = (hi - lo + TM - 1) / TM;
        if (tile < tiles) {
            m0 = lo + tile * TM;
            m_end = hi;
            break;
        }
        tile -= tiles;
    }
    if (e >= experts) return;
    const int n0 = blockIdx.x * TN;
    for (int r = threadIdx.x; r < TM; r += 128) {
        const int m = m0 + r;
        sm.a_rows[r] = m < m_end ? A + static_cast<size_t>(row_map ? row_map[m] : m) * lda : nullptr;
    }
    __syncthreads();
    float acc[2][4][4];
    mma_tile_64x64(sm, W + static_cast<size_t>(e) * N * K, K, 1, n0, N, K, acc);
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int m = m0 + tile_row(i, x), n = n0 + tile_col(j, x);
                if (m >= m_end || n >= N) continue;
                if (act >= 2) {             // elements 0 and 2 of a fragment are gates, their neighbours the ups
                    if (!(x & 1) && n + 1 < N)
                        C[static_cast<size_t>(m) * ldc + n / 2] = from_f32<TC>(gated_pair(act, acc[i][j][x], acc[i][j][x + 1], limit, alpha));
                    continue;
                }
                float v = acc[i][j][x];
                if (act == 1) {
                    v = fmaxf(v, 0.f);
                    v *= v;
                }
                C[static_cast<size_t>(m) * ldc + n] = from_f32<TC>(v);
            }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ Y, const int32_t* __restrict__ row_of, const float* __restrict__ weights,
                   const T* __restrict__ shared, const float* __restrict__ shared_gate, int gate_stride, T* __restrict__ out, int hidden,
                   int top) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const float share = shared_gate ? 1.f / (1.f + expf(-shared_gate[static_cast<size_t>(t) * gate_stride])) : 1.f;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < hidden; c += gridDim.y * blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int row = row_of[static_cast<size_t>(t) * top + k];
            if (row >= 0) acc = fmaf(weights[static_cast<size_t>(t) * top + k], Y[static_cast<size_t>(row) * hidden + c], acc);
        }
        if (shared) acc = fmaf(share, to_f32(shared[static_cast<size_t>(t) * hidden + c]), acc);
        out[static_cast<size_t>(t) * hidden + c] = from_f32<T>(acc);
    }
}

// relu(x)^2 in place, for the shared expert (the routed experts apply it in their product's epilogue)
template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ x, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float v = fmaxf(to_f32(x[i]), 0.f);
        x[i] = from_f32<T>(v * v);
    }
}

}  // namespace stride

using namespace stride;

extern "C" {

int stride_moe_route(const void* h, const void* w_router, const float* bias, const int32_t* seq_of_token, int32_t* ids, float* weights,
                     int tokens, int hidden, int experts, int top, int dtype, cudaStream_t stream) {
    if (tokens < 0 || hidden <= 0 || experts <= 0 || top <= 0 || top > experts) return STRIDE_BAD_ARGUMENT;
    if (experts > kMaxExperts || top > kMaxTop) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    const dim3 grid((tokens + 3) / 4);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(moe_route_kernel<float>, grid, dim3(128), 0, stream, static_cast<const float*>(h), static_cast<const float*>(w_router),
                       bias, seq_of_token, ids, weights, tokens, hidden, experts, top);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(moe_route_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(h),
                       static_cast<const __nv_bfloat16*>(w_router), bias, seq_of_token, ids, weights, tokens, hidden, experts, top);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_moe_select(const float* logits, const float* bias, const int32_t* seq_of_token, int32_t* ids, float* weights, int tokens,
                      int experts, int top, cudaStream_t stream) {
    if (tokens < 0 || experts <= 0 || top <= 0 || top > experts) return STRIDE_BAD_ARGUMENT;
    if (experts > kMaxExperts || top > kMaxTop) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    stride::launch(moe_select_kernel, dim3((tokens + 3) / 4), dim3(128), 0, stream, logits, bias, seq_of_token, ids, weights, tokens, experts, top);
    return STRIDE_LAUNCH_STATUS();
}

int stride_moe_select_groups(const float* logits, int ld, const float* correction, const int32_t* seq_of_token, int32_t* ids,
                             float* weights, int tokens, int experts, int top, int groups, int keep, float route_scale, int rule,
                             cudaStream_t stream) {
    if (tokens < 0 || experts <= 0 || top <= 0 || top > experts || ld < experts || groups <= 0 || keep <= 0 || keep > groups ||
        experts % groups || top > keep * (experts / groups) || rule < 0 || rule > 7)
        return STRIDE_BAD_ARGUMENT;
    if (experts > kMaxExperts || top > kMaxTop) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    stride::launch(moe_select_sigmoid_kernel, dim3((tokens + 3) / 4), dim3(128), 0, stream, logits, ld, correction, seq_of_token, ids, weights,
                   tokens, experts, top, groups, keep, route_scale, rule);
    return STRIDE_LAUNCH_STATUS();
}

int stride_moe_select_sigmoid(const float* logits, int ld, const float* correction, const int32_t* seq_of_token, int32_t* ids,
                              float* weights, int tokens, int experts, int top, int groups, int keep, float route_scale, cudaStream_t stream) {
    return stride_moe_select_groups(logits, ld, correction, seq_of_token, ids, weights, tokens, experts, top, groups, keep, route_scale, 0, stream);
}

int stride_moe_plan(const int32_t* ids, int tokens, int top, int experts, int32_t* offsets, int32_t* perm_token, int32_t* row_of,
                    int32_t* rank_tmp, cudaStream_t stream) {
    if (tokens < 0 || top <= 0 || experts <= 0) return STRIDE_BAD_ARGUMENT;
    if (experts > kMaxExperts) return STRIDE_UNSUPPORTED;
    stride::launch(moe_plan_kernel, dim3(1), dim3(256), 0, stream, ids, tokens * top, experts, offsets, perm_token, row_of, rank_tmp, top);
    return STRIDE_LAUNCH_STATUS();
}

// kind: 0 = everything float32 (FMA); 1 = bfloat16 A and W, bfloat16 C; 2 = bfloat16 A and W, float32 C (both on the
// tensor cores); 3 = as 2 on the FMA kernel.
int stride_grouped_gemm(const void* A, int lda, const int32_t* row_map, const void* W, const int32_t* offsets, int experts, void* C,
                        int ldc, int max_rows, int N, int K, int act, float limit, float alpha, int kind, cudaStream_t stream) {
    if (max_rows < 0 || experts <= 0 || N <= 0 || K <= 0 || lda < K || act < 0 || act > 3 || ldc < (act >= 2 ? N / 2 : N) || (act >= 2 && N % 2))
        return STRIDE_BAD_ARGUMENT;
    if (max_rows == 0) return 0;
    const int max_tiles = (max_rows + GM - 1) / GM + experts;       // no expert has more than one ragged tile
    if (max_tiles > 65535) return STRIDE_UNSUPPORTED;
    const dim3 grid((N + GN - 1) / GN, max_tiles);
    static_assert(GM == TM && GN == TN, "both forms of the grouped product use tiles of one size");
    if (kind == 1)
        stride::launch(grouped_gemm_tc_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(A), lda, row_map,
                       static_cast<const __nv_bfloat16*>(W), offsets, experts, static_cast<__nv_bfloat16*>(C), ldc, N, K, act, limit, alpha);
    else if (kind == 2)
        stride::launch(grouped_gemm_tc_kernel<float>, grid, dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(A), lda, row_map,
                       static_cast<const __nv_bfloat16*>(W), offsets, experts, static_cast<float*>(C), ldc, N, K, act, limit, alpha);
    else if (kind == 3)     // bfloat16 operands on the FMA kernel (kept for comparison)
        stride::launch(grouped_gemm_kernel<__nv_bfloat16, __nv_bfloat16, float>, grid, dim3(256), 0, stream,
                       static_cast<const __nv_bfloat16*>(A), lda, row_map, static_cast<const __nv_bfloat16*>(W), offsets, experts,
                       static_cast<float*>(C), ldc, N, K, act, limit, alpha);
    else if (kind == 0)
        stride::launch(grouped_gemm_kernel<float, float, float>, grid, dim3(256), 0, stream, static_cast<const float*>(A), lda, row_map,
                       static_cast<const float*>(W), offsets, experts, static_cast<float*>(C), ldc, N, K, act, limit, alpha);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_moe_combine(const float* Y, const int32_t* row_of, const float* weights, const void* shared, const float* shared_gate,
                       int gate_stride, void* out, int tokens, int hidden, int top, int dtype, cudaStream_t stream) {
    if (tokens < 0 || hidden <= 0 || top <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const dim3 grid(tokens, hidden >= 2048 ? 4 : 1);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(moe_combine_kernel<float>, grid, dim3(256), 0, stream, Y, row_of, weights, static_cast<const float*>(shared),
                       shared_gate, gate_stride, static_cast<float*>(out), hidden, top);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(moe_combine_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, Y, row_of, weights,
                       static_cast<const __nv_bfloat16*>(shared), shared_gate, gate_stride, static_cast<__nv_bfloat16*>(out), hidden, top);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_relu_squared(void* x, long long n, int dtype, cudaStream_t stream) {
    if (n < 0) return STRIDE_BAD_ARGUMENT;
    if (n == 0) return 0;
    const unsigned blocks = static_cast<unsigned>(n / 256 >= 4096 ? 4096 : (n + 255) / 256);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(relu_squared_kernel<float>, dim3(blocks), dim3(256), 0, stream, static_cast<float*>(x), static_cast<size_t>(n));
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(relu_squared_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, static_cast<__nv_bfloat16*>(x), static_cast<size_t>(n));
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
