// The matrix memory of xLSTM (Beck et al., "xLSTM: Extended Long Short-Term Memory"): per head a matrix S [D, DV], a
// vector n [D] and a running maximum m, all float32, updated once a token:
//
//   li = c tanh((z_i + b_i) / c)                      log of the input gate, capped at c
//   lf = logsigmoid(c tanh((z_f + b_f) / c))          log of the forget gate
//   m' = max(lf + m, li)
//   S' = exp(lf + m - m') S + exp(li - m') k v^T ;  n' likewise with k alone
//   o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
//
// m starts at zero (a cleared state row), not at minus infinity. The memory is independent over the DV columns of S; along a
// column the only coupling is the sum over D of a read. A column belongs to 8 or 16 neighbouring lanes, lane l holding rows
// l, l + lanes, ... in registers together with the same rows of n (every column's lanes keep n for themselves: a few more
// multiply-adds a token, and no exchange between columns). A CTA of 128 threads owns 16 or 8 columns of one head of one
// request and walks the request's tokens of the step in order; the inputs of 16 (or 8) tokens are staged in shared memory at a time
// (q already times `q_scale`, the two gate logarithms computed once a token). The order of every sum depends on the token
// only, so a token's output is bitwise the same in a whole prompt, in portions or decoded alone.
//
// State row of a request: S [H, D, DV], then n [H, D], then m [H].
#include "common.cuh"

namespace stride {

constexpr int kLstmThreads = 128;

struct LstmArgs {
    const void* proj;       // [tokens, ld] in the compute type: q of head h at q_off + h * D, k at k_off + h * D, v at v_off + h * DV
    int ld, q_off, k_off, v_off;
    const float* gates;     // [tokens, ld_gates] float32: column h the input gate's projection, column H + h the forget gate's
    int ld_gates;
    const float* bias_i;    // [H]
    const float* bias_f;    // [H]
    float cap, q_scale;
    float* o;               // [tokens, H * DV] float32
    float* state;           // [slots, state_stride]
    long long state_stride;
    const int32_t* q_start;
    const int32_t* q_len;
    const int32_t* state_slot;
    int H, D, DV;
};

__device__ __forceinline__ float log_sigmoid_f(float z) { return z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z)); }

// LANES lanes share a column, each with R of its rows: D <= LANES * R. What is carried from token to token is one
// multiply-add an entry of S and n and two operations on m; everything else of a token (its exponentials, the sums over the
// lanes, the division) hangs off that chain. So:
// * the inputs of the next chunk are fetched into registers (all loads at once, no branch between them) before the current
//   chunk is worked through, and stored into the other shared-memory buffer afterwards;
// * while they are stored, warp 0 follows m through that chunk (lane t holds token t's two gate logarithms; sixteen steps of
//   max and add in token order, the operands handed round by shuffles) and its lanes make the three exponentials of a token
//   each, so the loop over a chunk reads them from shared memory;
// * that loop always runs its full length (tokens past the request's end keep the memory as it is) and is unrolled, so that
//   the sums, shuffles and divisions of one token stand beside the multiply-adds of the next ones; a lane's rows come in
//   groups of four neighbours, one 16-byte read of shared memory a group; the quotient is a product with the hardware's
//   reciprocal (2 units in the last place; the same instruction for every cutting).
template <typename T, int LANES, int R, int CHUNK = 16>
__global__ void __launch_bounds__(kLstmThreads)
mlstm_scan_kernel(const LstmArgs p) {
    constexpr int DP = R * LANES;
    constexpr int COLS = kLstmThreads / LANES;
    constexpr int ROW_ITEMS = CHUNK * DP / kLstmThreads;
    constexpr int V_ITEMS = (CHUNK * COLS + kLstmThreads - 1) / kLstmThreads;
    static_assert((CHUNK * DP) % kLstmThreads == 0 && CHUNK <= 32, "chunks are shared out evenly");
    constexpr bool QUADS = R % 4 == 0;      // a lane's rows in groups of four neighbours: one 16-byte read of shared memory a group
    __shared__ __align__(16) float s_q[2][CHUNK][DP], s_k[2][CHUNK][DP];
    __shared__ float s_v[2][CHUNK][COLS];
    __shared__ float s_keep[2][CHUNK], s_take[2][CHUNK], s_floor[2][CHUNK];
    const int seq = blockIdx.z, h = blockIdx.y;
    const int len = p.q_len[seq];
    if (len <= 0) return;
    const int start = p.q_start[seq];
    const int il = threadIdx.x & (LANES - 1), jc = threadIdx.x / LANES;
    const int j = blockIdx.x * COLS + jc;
    const int H = p.H, D = p.D, DV = p.DV;
    const T* proj = static_cast<const T*>(p.proj);
    float* base = p.state + static_cast<size_t>(p.state_slot[seq]) * p.state_stride;
    float* S_g = base + static_cast<size_t>(h) * D * DV;
    float* n_g = base + static_cast<size_t>(H) * D * DV + static_cast<size_t>(h) * D;
    float* m_g = base + static_cast<size_t>(H) * D * DV + static_cast<size_t>(H) * D + h;
    // lane il of a column's lanes holds the rows 4 LANES g + 4 il + e (g < R / 4, e < 4), or il + LANES r where R is no multiple of 4
    auto row_of = [&](int r) { return QUADS ? 4 * LANES * (r >> 2) + 4 * il + (r & 3) : il + LANES * r; };
    float S[R], nn[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = row_of(r);
        S[r] = (i < D && j < DV) ? S_g[static_cast<size_t>(i) * DV + j] : 0.f;
        nn[r] = i < D ? n_g[i] : 0.f;
    }
    float m = *m_g;             // followed by warp 0 only
    const float bias_i = p.bias_i[h], bias_f = p.bias_f[h];

    float fq[ROW_ITEMS], fk[ROW_ITEMS], fv[V_ITEMS], zi = 0.f, zf = 0.f;
    auto fetch = [&](int c0) {      // the chunk from local token c0 on, into registers (zeros past the request's end)
#pragma unroll
        for (int n = 0; n < ROW_ITEMS; ++n) {
            const int idx = n * kLstmThreads + threadIdx.x;
            const int tt = idx / DP, i = idx - tt * DP;
            const bool on = c0 + tt < len && i < D;
            const size_t row = static_cast<size_t>(start + (on ? c0 + tt : 0)) * p.ld + h * D + (on ? i : 0);
            const float q = to_f32(proj[row + p.q_off]), k = to_f32(proj[row + p.k_off]);
            fq[n] = on ? q * p.q_scale : 0.f;
            fk[n] = on ? k : 0.f;
        }
#pragma unroll
        for (int n = 0; n < V_ITEMS; ++n) {
            const int idx = n * kLstmThreads + threadIdx.x;
            const int tt = idx / COLS, c = idx - tt * COLS;
            const int col = blockIdx.x * COLS + c;
            const bool on = tt < CHUNK && c0 + tt < len && col < DV;
            const float v = to_f32(proj[static_cast<size_t>(start + (on ? c0 + tt : 0)) * p.ld + p.v_off + h * DV + (on ? col : 0)]);
            fv[n] = on ? v : 0.f;
        }
        if (threadIdx.x < CHUNK) {
            const bool on = c0 + static_cast<int>(threadIdx.x) < len;
            const size_t row = static_cast<size_t>(start + (on ? c0 + threadIdx.x : 0)) * p.ld_gates;
            zi = p.gates[row + h];
            zf = p.gates[row + H + h];
        }
    };
    auto stash = [&](int buf, int c0) {
#pragma unroll
        for (int n = 0; n < ROW_ITEMS; ++n) {
            const int idx = n * kLstmThreads + threadIdx.x;
            const int tt = idx / DP, i = idx - tt * DP;
            s_q[buf][tt][i] = fq[n];
            s_k[buf][tt][i] = fk[n];
        }
#pragma unroll
        for (int n = 0; n < V_ITEMS; ++n) {
            const int idx = n * kLstmThreads + threadIdx.x;
            if (idx < CHUNK * COLS) s_v[buf][idx / COLS][idx % COLS] = fv[n];
        }
        if (threadIdx.x < 32) {     // warp 0: the gates of the chunk's tokens and the chain of m through them
            const int lane = threadIdx.x;
            const bool live = lane < CHUNK && c0 + lane < len;
            // a token past the end leaves m as it is: max(0 + m, -inf)
            const float li = live ? p.cap * tanhf((zi + bias_i) / p.cap) : -INFINITY;
            const float lf = live ? log_sigmoid_f(p.cap * tanhf((zf + bias_f) / p.cap)) : 0.f;
            float m_before = 0.f, m_after = 0.f;
#pragma unroll
            for (int tt = 0; tt < CHUNK; ++tt) {
                const float m_new = fmaxf(__shfl_sync(0xffffffffu, lf, tt) + m, __shfl_sync(0xffffffffu, li, tt));
                if (lane == tt) { m_before = m; m_after = m_new; }
                m = m_new;
            }
            if (lane < CHUNK) {
                s_keep[buf][lane] = live ? expf(lf + m_before - m_after) : 1.f;
                s_take[buf][lane] = live ? expf(li - m_after) : 0.f;
                s_floor[buf][lane] = live ? expf(-m_after) : 1.f;
            }
        }
    };

    fetch(0);
    stash(0, 0);
    __syncthreads();
    int buf = 0;
    for (int c0 = 0; c0 < len; c0 += CHUNK, buf ^= 1) {
        const int nt = min(CHUNK, len - c0);
        const bool more = c0 + CHUNK < len;
        if (more) fetch(c0 + CHUNK);
#pragma unroll 4
        for (int tt = 0; tt < CHUNK; ++tt) {
            const float keep = s_keep[buf][tt], take = s_take[buf][tt];
            const float vj = s_v[buf][tt][jc] * take;
            float acc[4] = {0.f, 0.f, 0.f, 0.f}, den[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (QUADS) {
                const float4* k4 = reinterpret_cast<const float4*>(&s_k[buf][tt][4 * il]);
                const float4* q4 = reinterpret_cast<const float4*>(&s_q[buf][tt][4 * il]);
#pragma unroll
                for (int g = 0; g < R / 4; ++g) {
                    const float4 kv = k4[LANES * g], qv = q4[LANES * g];
                    const float kk[4] = {kv.x, kv.y, kv.z, kv.w}, qq[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        S[4 * g + e] = fmaf(keep, S[4 * g + e], kk[e] * vj);
                        nn[4 * g + e] = fmaf(keep, nn[4 * g + e], take * kk[e]);
                        acc[e] = fmaf(S[4 * g + e], qq[e], acc[e]);
                        den[e] = fmaf(nn[4 * g + e], qq[e], den[e]);
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float kk = s_k[buf][tt][il + LANES * r], qq = s_q[buf][tt][il + LANES * r];
                    S[r] = fmaf(keep, S[r], kk * vj);
                    nn[r] = fmaf(keep, nn[r], take * kk);
                    acc[r & 3] = fmaf(S[r], qq, acc[r & 3]);
                    den[r & 3] = fmaf(nn[r], qq, den[r & 3]);
                }
            }
            float num = (acc[0] + acc[1]) + (acc[2] + acc[3]), dot = (den[0] + den[1]) + (den[2] + den[3]);
#pragma unroll
            for (int o = 1; o < LANES; o <<= 1) {
                num += __shfl_xor_sync(0xffffffffu, num, o);
                dot += __shfl_xor_sync(0xffffffffu, dot, o);
            }
            if (il == 0 && j < DV && tt < nt)
                p.o[(static_cast<size_t>(start + c0 + tt) * H + h) * DV + j] = __fdividef(num, fmaxf(fabsf(dot), s_floor[buf][tt]) + 1e-6f);
        }
        if (more) stash(buf ^ 1, c0 + CHUNK);      // nobody reads that buffer: its chunk was finished before the last barrier
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = row_of(r);
        if (i < D && j < DV) S_g[static_cast<size_t>(i) * DV + j] = S[r];
        if (blockIdx.x == 0 && jc == 0 && i < D) n_g[i] = nn[r];
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *m_g = m;
}

}  // namespace stride

using namespace stride;

extern "C" {

// One launch for every request of the step (grid z: the step's sequence slots, empty ones return at once).
int stride_mlstm_scan(const void* proj, int ld, int q_off, int k_off, int v_off, const float* gates, int ld_gates, const float* bias_i,
                      const float* bias_f, float cap, float q_scale, float* o, float* state, long long state_stride,
                      const int32_t* q_start, const int32_t* q_len, const int32_t* state_slot, int num_seqs, int H, int D, int DV,
                      int dtype, cudaStream_t stream) {
    if (num_seqs < 0 || H <= 0 || D <= 0 || DV <= 0 || ld <= 0 || ld_gates < 2 * H || !(cap > 0.f) || q_off < 0 || k_off < 0 || v_off < 0)
        return STRIDE_BAD_ARGUMENT;
    if (dtype != STRIDE_DTYPE_F32 && dtype != STRIDE_DTYPE_BF16) return STRIDE_BAD_ARGUMENT;
    if (state_stride < static_cast<long long>(H) * D * DV + static_cast<long long>(H) * D + H) return STRIDE_BAD_ARGUMENT;
    if (D > 256 || H > 65535 || num_seqs > 65535) return STRIDE_UNSUPPORTED;
    if (num_seqs == 0) return 0;
    LstmArgs a;
    a.proj = proj; a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
    a.gates = gates; a.ld_gates = ld_gates; a.bias_i = bias_i; a.bias_f = bias_f; a.cap = cap; a.q_scale = q_scale;
    a.o = o; a.state = state; a.state_stride = state_stride; a.q_start = q_start; a.q_len = q_len; a.state_slot = state_slot;
    a.H = H; a.D = D; a.DV = DV;
    const dim3 block(kLstmThreads);
    // a chain of tokens keeps few CTAs busy for long: launched without an early start behind the kernel before it.
    // Heads of up to 32 rows: 8 lanes a column; larger ones 16 lanes, so that a lane holds at most 16 rows.
    auto run = [&](auto kernel, int lanes) {
        const int cols = kLstmThreads / lanes;
        stride::launch_alone(kernel, dim3((DV + cols - 1) / cols, H, num_seqs), block, 0, stream, a);
    };
    if (dtype == STRIDE_DTYPE_BF16) {
        if (D <= 16) run(mlstm_scan_kernel<__nv_bfloat16, 8, 2>, 8);
        else if (D <= 32) run(mlstm_scan_kernel<__nv_bfloat16, 8, 4>, 8);
        else if (D <= 64) run(mlstm_scan_kernel<__nv_bfloat16, 16, 4>, 16);
        else if (D <= 128) run(mlstm_scan_kernel<__nv_bfloat16, 16, 8>, 16);
        else run(mlstm_scan_kernel<__nv_bfloat16, 16, 16, 8>, 16);        // chunks of 8 tokens: two buffers of 16 would not fit
    } else {
        if (D <= 16) run(mlstm_scan_kernel<float, 8, 2>, 8);
        else if (D <= 32) run(mlstm_scan_kernel<float, 8, 4>, 8);
        else if (D <= 64) run(mlstm_scan_kernel<float, 16, 4>, 16);
        else if (D <= 128) run(mlstm_scan_kernel<float, 16, 8>, 16);
        else run(mlstm_scan_kernel<float, 16, 16, 8>, 16);
    }
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
