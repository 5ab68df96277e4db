// Mixers that keep a matrix per head as their memory: S [D, DV] in float32, updated once a token by a rank-one term and
// read with a query. Two rules:
//
//   gated delta rule     S <- diag(g_t) S ;  u = beta_t (v_t - S^T k_t) ;  S <- S + k_t u^T ;  o_t = S^T q_t
//                        (Yang, Kautz, Hatamizadeh, "Gated Delta Networks: Improving Mamba2 with Delta Rule"; here the
//                        decay g_t is a vector over the D key channels)
//   decayed memory with a bonus (the time mixing of RWKV-6: Peng et al., "Eagle and Finch: RWKV with Matrix-Valued
//                        States and Dynamic Recurrence")
//                        o_t = (S + diag(b) k_t v_t^T)^T r_t ;  S <- diag(w_t) S + k_t v_t^T
//
// Both are independent over the DV columns of S, and along a column the only coupling is one sum over D per read. The
// scan kernel gives a column to 4, 8 or 16 neighbouring lanes: each holds R of the rows in registers (groups of four
// neighbouring rows; rows beyond D carry zeros), sums its part in four partial sums and the lanes add up by shuffles,
// always in the same order. A CTA of 128 threads owns 32, 16 or 8 columns of one head of one request and walks the
// request's tokens of the step in order; the inputs of 8 or 16 tokens are staged in shared memory at a time, the next ones
// being fetched into registers meanwhile. The order of every sum depends on the token
// only, so a token's output is bitwise the same in a whole prompt, in portions or decoded alone. State per request lives
// in one float32 row of the mixer's state tensor: S [heads, D, DV], then whatever the mixer needs of the past inputs.
//
// Kernels around the scans:
//   delta_prepare   per token: causal convolution (taps from the state's tail at a portion's start) and SiLU of the q, k
//                   and v projections, unit length for q and k per head (q also times D^-1/2), beta = sigmoid, and the
//                   decay exp(-exp(A_log) softplus(a + dt_bias)); everything float32
//   shift_mix       per token: the lerps between a token's input and the previous token's (the state's at a portion's
//                   start), one per consumer; the portion's last input goes into the state
//   head_norm_gate  o / rms(o) * weight * gate per head, into the compute type for the output projection
// The scans end by writing S back and, for the delta rule, by moving the convolution's tail in the state forward.
#include "common.cuh"

namespace stride {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

__device__ __forceinline__ float load_any(const void* p, size_t i, int is_bf16) {
    return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]) : static_cast<const float*>(p)[i];
}

// ------------------------------------------------------------------------------------------------ delta_prepare
// proj [tokens, ld] (compute type): columns [0, GD) q, [GD, 2GD) k, [2GD, 2GD + HV) v, then H columns of beta's
// projection. conv_w [C, taps] float32 for the C = 2GD + HV channels in the same order. low [tokens, ld_low] float32:
// columns [0, HD) the decay's projection. tail: the state's rows [taps - 1, C] at `tail_off` floats into a slot's row.
// Outputs float32: qk [tokens, 2GD] (q then k, unit length), v [tokens, HV], beta [tokens, H], decay [tokens, HD].
// What is handed on of a decay g is g - 1 = expm1(log g), and the scans compute S + (g - 1) S: for a channel that forgets
// slowly g is within 1e-4 of 1, where float32 has steps of 6e-8 and a rounded g costs a little with every token.
// One warp a head: warps 0..2G-1 the q and k heads, then H warps for the v heads, which also do beta and the decay.
constexpr int kPrepWarps = 8;
constexpr int kMaxPerLane = 8;      // head sizes up to 256

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
delta_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ conv_w, const float* __restrict__ low, int ld_low,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ state,
                     long long state_stride, long long tail_off, const int32_t* __restrict__ seq_of_token,
                     const int32_t* __restrict__ q_start, const int32_t* __restrict__ state_slot, float* __restrict__ qk,
                     float* __restrict__ v_out, float* __restrict__ beta, float* __restrict__ decay, int G, int H, int D, int DV,
                     int taps, float unit_eps) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * kPrepWarps + warp;
    if (head >= 2 * G + H) return;
    const int GD = G * D, HV = H * DV, C = 2 * GD + HV;
    const bool is_v = head >= 2 * G;
    const int n = is_v ? DV : D;
    const int c0 = is_v ? 2 * GD + (head - 2 * G) * DV : head * D;       // first channel of this head
    const int seq = seq_of_token[t];
    float* dst = is_v ? v_out + static_cast<size_t>(t) * HV + (head - 2 * G) * DV : qk + static_cast<size_t>(t) * 2 * GD + head * D;
    if (seq < 0) {          // a padded row of a fixed-size batch
        for (int e = lane; e < n; e += 32) dst[e] = 0.f;
        if (is_v) {
            const int h = head - 2 * G;
            for (int e = lane; e < D; e += 32) decay[static_cast<size_t>(t) * H * D + h * D + e] = 0.f;
            if (lane == 0) beta[static_cast<size_t>(t) * H + h] = 0.f;
        }
        return;
    }
    const int start = q_start[seq];
    const int local = t - start;
    const float* tail = state + static_cast<size_t>(state_slot[seq]) * state_stride + tail_off;
    float y[kMaxPerLane];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
        const int e = lane + 32 * r;
        y[r] = 0.f;
        if (e < n) {
            const int c = c0 + e;
            float acc = 0.f;
            for (int j = 0; j < taps; ++j) {
                const int src = local - (taps - 1) + j;
                const float x = src >= 0 ? to_f32(proj[static_cast<size_t>(start + src) * ld + c])
                                         : tail[static_cast<size_t>(taps - 1 + src) * C + c];
                acc = fmaf(conv_w[static_cast<size_t>(c) * taps + j], x, acc);
            }
            y[r] = silu_f(acc);
            ss = fmaf(y[r], y[r], ss);
        }
    }
    float mult = 1.f;
    if (!is_v) {
        ss = warp_sum(ss);
        mult = 1.f / sqrtf(ss + unit_eps);
        if (head < G) mult *= 1.f / sqrtf(static_cast<float>(D));
    }
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
        const int e = lane + 32 * r;
        if (e < n) dst[e] = y[r] * mult;
    }
    if (is_v) {
        const int h = head - 2 * G;
        const float rate = expf(a_log[h]);
        for (int e = lane; e < D; e += 32) {
            const float a = low[static_cast<size_t>(t) * ld_low + h * D + e] + dt_bias[h * D + e];
            decay[static_cast<size_t>(t) * H * D + h * D + e] = expm1f(-rate * softplus_f(a));
        }
        if (lane == 0) beta[static_cast<size_t>(t) * H + h] = sigmoid_f(to_f32(proj[static_cast<size_t>(t) * ld + C + h]));
    }
}

// ---------------------------------------------------------------------------------------------------- shift_mix
// x [tokens, width] (compute type); mu [mixes, width] float32; out [mixes, tokens, width] (compute type):
// out[s, t] = x[t] + (prev - x[t]) * mu[s], prev = x[t - 1] inside a portion and the state's vector at its start. The CTA
// of a portion's first token then stores the portion's last input as the new state (it alone touches the state).
template <typename T>
__global__ void __launch_bounds__(256)
shift_mix_kernel(const T* __restrict__ x, const float* __restrict__ mu, float* __restrict__ state, long long state_stride,
                 long long prev_off, const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ q_start,
                 const int32_t* __restrict__ q_len, const int32_t* __restrict__ state_slot, T* __restrict__ out, int tokens, int width,
                 int mixes) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0) {
        for (int c = threadIdx.x; c < width; c += blockDim.x)
            for (int s = 0; s < mixes; ++s) out[(static_cast<size_t>(s) * tokens + t) * width + c] = from_f32<T>(0.f);
        return;
    }
    const int start = q_start[seq];
    const bool first = t == start;
    float* prev_state = state + static_cast<size_t>(state_slot[seq]) * state_stride + prev_off;
    const T* last = x + static_cast<size_t>(start + q_len[seq] - 1) * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float cur = to_f32(x[static_cast<size_t>(t) * width + c]);
        const float prev = first ? prev_state[c] : to_f32(x[static_cast<size_t>(t - 1) * width + c]);
        const float d = prev - cur;
        for (int s = 0; s < mixes; ++s)
            out[(static_cast<size_t>(s) * tokens + t) * width + c] = from_f32<T>(fmaf(d, mu[static_cast<size_t>(s) * width + c], cur));
        if (first) prev_state[c] = to_f32(last[c]);
    }
}

// ------------------------------------------------------------------------------------------------ head_norm_gate
// o [tokens, H, DV] float32 -> out [tokens, H * DV] (compute type): o / sqrt(mean(o^2) + eps) * weight * gate.
// weight [.. ] float32 read at h * w_head_stride + j (0: one weight for all heads). gate_kind 0: sigmoid of float32
// gate[t * ld_gate + h * DV + j]; 1: silu of a compute-type gate at the same place; 2: sigmoid of a compute-type gate.
// One warp a (token, head).
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ weight, int w_head_stride, const void* __restrict__ gate,
                      int ld_gate, int gate_kind, T* __restrict__ out, int tokens, int H, int DV, float eps) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long pair = static_cast<long long>(blockIdx.x) * 8 + warp;
    if (pair >= static_cast<long long>(tokens) * H) return;
    const int t = static_cast<int>(pair / H), h = static_cast<int>(pair % H);
    const float* row = o + (static_cast<size_t>(t) * H + h) * DV;
    float ss = 0.f;
    for (int j = lane; j < DV; j += 32) ss = fmaf(row[j], row[j], ss);
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / static_cast<float>(DV) + eps);
    for (int j = lane; j < DV; j += 32) {
        const size_t at = static_cast<size_t>(t) * ld_gate + h * DV + j;
        const float g = gate_kind == 0   ? sigmoid_f(static_cast<const float*>(gate)[at])
                        : gate_kind == 1 ? silu_f(to_f32(static_cast<const T*>(gate)[at]))
                                         : sigmoid_f(to_f32(static_cast<const T*>(gate)[at]));
        out[(static_cast<size_t>(t) * H + h) * DV + j] = from_f32<T>(row[j] * inv * weight[h * w_head_stride + j] * g);
    }
}

// --------------------------------------------------------------------------------------------------------- scans
constexpr int kScanThreads = 128;

struct ScanArgs {
    const void* a;          // queries (delta) / receptance (memory with bonus): [tokens, lda], head h at column (h / group) * D
    const void* k;          // keys, the same layout
    const float* w;         // [tokens, H * D]: the decay minus one (delta), or its double logarithm before w0 (bonus rule)
    const void* v;          // values [tokens, ldv], head h at column h * DV
    const float* beta;      // [tokens, H] (delta) or null
    const float* w0;        // [H * D] added to w before exp(-exp(.)) (bonus rule) or null
    const float* bonus;     // [H * D] (bonus rule) or null
    float* o;               // [tokens, H * DV] float32
    float* state;           // [slots, state_stride]; S of head h at h * D * DV
    long long state_stride;
    const int32_t* q_start;
    const int32_t* q_len;
    const int32_t* state_slot;
    int lda, ldv, H, group, D, DV, in_bf16;
    // the convolution's tail (delta rule; taps 0: none): the last taps - 1 rows of proj's first C columns
    const void* proj;
    int ld_proj, C, taps, proj_bf16;
    long long tail_off;
    // pieces (mode 0: none, a request's tokens in one chain). A piece is `piece` consecutive tokens of a request; grid z is
    // request * max_pieces + piece. Mode 1 runs every piece from a zero memory, writes no output, and leaves the piece's
    // memory in piece_s [z, H, D, DV] and the product of its decays in piece_p [z, H, D]; mode 2 runs every piece from
    // piece_s (by then the memory at the piece's start), writes the outputs and leaves the state alone.
    // init (mode 1): 1 starts every column from zero, 2 from the unit matrix (column j holds a one in row j): with no values
    // (v null) the memory of a piece then ends as the matrix that carries any memory across the piece.
    int mode, piece, max_pieces, init;
    float* piece_s;
    float* piece_p;
};

// LANES lanes share a column, each with R of its rows (R a multiple of 4): D <= LANES * R. A thread works on NC columns
// at once (COLS apart), CHUNK tokens are staged at a time. One token follows the other and a warp issues in order, so what
// sets the pace of a prompt is the chain of dependent instructions a token costs a warp (shared-memory reads, the sums,
// the shuffles), not the amount of arithmetic: the rows are spread over as many lanes as the head size allows, and the NC
// columns of a thread are independent chains that fill one another's waits (they also share the reads of k, q and the decay).
// PIECES false: the one chain only (mode 0), with nothing of the pieces' bookkeeping in its loop.
template <int LANES, int R, int NC, int CHUNK, int RULE, bool PIECES>      // RULE 0: gated delta rule, 1: decayed memory with a bonus
__global__ void __launch_bounds__(kScanThreads)
scan_kernel(const ScanArgs p) {
    // Launched without programmatic dependent launch (launch_alone): no trigger, and nothing to wait for.
    const int mode = PIECES ? p.mode : 0;
    constexpr int DP = R * LANES;                           // rows with padding
    constexpr int THREADS = kScanThreads;
    constexpr int COLS = THREADS / LANES;                   // columns of one pass over the threads
    constexpr int CTA_COLS = COLS * NC;                     // columns of this CTA
    constexpr int ROW_ITEMS = CHUNK * DP / THREADS;         // entries of each [chunk, DP] array a thread fetches
    constexpr int V_ITEMS = (CHUNK * CTA_COLS + THREADS - 1) / THREADS;
    static_assert(R % 4 == 0 && (CHUNK * DP) % THREADS == 0 && CHUNK <= THREADS, "chunks are shared out evenly");
    // two buffers: while the tokens of one chunk are worked through, the next chunk's inputs are on their way from
    // global memory into registers; they are stored (the decay's exponentials applied) when the chunk is done
    __shared__ __align__(16) float s_a[2][CHUNK][DP], s_k[2][CHUNK][DP], s_w[2][CHUNK][DP];
    __shared__ float s_v[2][CHUNK][CTA_COLS], s_beta[2][CHUNK];
    __shared__ __align__(16) float s_bonus[DP], s_w0[DP];
    const int seq = mode ? blockIdx.z / p.max_pieces : blockIdx.z, h = blockIdx.y;
    const int first = mode ? (blockIdx.z % p.max_pieces) * p.piece : 0;         // this CTA's tokens of the request: [first, len)
    const int len = mode ? min(p.q_len[seq], first + p.piece) : p.q_len[seq];
    if (len <= first) return;
    const int start = p.q_start[seq];
    const int il = threadIdx.x & (LANES - 1), jc = threadIdx.x / LANES;
    const int j0 = blockIdx.x * CTA_COLS + jc;              // this thread's columns: j0 + c * COLS
    const int D = p.D, DV = p.DV, H = p.H;
    const int hk = h / p.group;
    float* S_g = mode ? p.piece_s + (static_cast<size_t>(blockIdx.z) * H + h) * D * DV
                        : p.state + static_cast<size_t>(p.state_slot[seq]) * p.state_stride + static_cast<size_t>(h) * D * DV;
    // lane il of a column's lanes holds rows 4 LANES g + 4 il + e (g < R / 4, e < 4) in S[.][4 g + e]: four neighbouring rows
    // are one 16-byte read of shared memory, and the lanes read consecutive 16 bytes
    auto row_of = [&](int r) { return 4 * LANES * (r >> 2) + 4 * il + (r & 3); };
    float S[NC][R];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = row_of(r), j = j0 + c * COLS;
            S[c][r] = mode == 1 ? ((p.init == 2 && i == j && i < D) ? 1.f : 0.f)
                                  : ((i < D && j < DV) ? S_g[static_cast<size_t>(i) * DV + j] : 0.f);
        }
    float decayed[R];           // mode 1: the product of the decays of this thread's rows over the piece
#pragma unroll
    for (int r = 0; r < R; ++r) decayed[r] = 1.f;
    if (RULE == 1)
        for (int i = threadIdx.x; i < DP; i += blockDim.x) {
            s_bonus[i] = i < D ? p.bonus[h * D + i] : 0.f;
            s_w0[i] = i < D ? p.w0[h * D + i] : 0.f;
        }

    float fa[ROW_ITEMS], fk[ROW_ITEMS], fw[ROW_ITEMS], fv[V_ITEMS], fb = 0.f;
    auto fetch = [&](int c0) {          // the chunk from token c0 on, into registers (zeros past the request's end)
#pragma unroll
        for (int n = 0; n < ROW_ITEMS; ++n) {
            const int idx = n * THREADS + threadIdx.x;
            const int tt = idx / DP, i = idx - tt * DP;
            fa[n] = fk[n] = fw[n] = 0.f;
            if (c0 + tt < len && i < D) {
                const size_t row = static_cast<size_t>(start + c0 + tt);
                fa[n] = load_any(p.a, row * p.lda + hk * D + i, p.in_bf16);
                fk[n] = load_any(p.k, row * p.lda + hk * D + i, p.in_bf16);
                fw[n] = p.w[row * H * D + h * D + i];
            }
        }
#pragma unroll
        for (int n = 0; n < V_ITEMS; ++n) {
            const int idx = n * THREADS + threadIdx.x;
            const int tt = idx / CTA_COLS, c = idx - tt * CTA_COLS;
            const int col = blockIdx.x * CTA_COLS + c;
            fv[n] = ((!PIECES || p.v != nullptr) && tt < CHUNK && c0 + tt < len && col < DV)
                        ? load_any(p.v, static_cast<size_t>(start + c0 + tt) * p.ldv + h * DV + col, p.in_bf16) : 0.f;
        }
        if (RULE == 0 && threadIdx.x < CHUNK)
            fb = c0 + threadIdx.x < len ? p.beta[static_cast<size_t>(start + c0 + threadIdx.x) * H + h] : 0.f;
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int n = 0; n < ROW_ITEMS; ++n) {
            const int idx = n * THREADS + threadIdx.x;
            const int tt = idx / DP, i = idx - tt * DP;
            float w = fw[n];
            if (RULE == 1) w = i < D ? expm1f(-expf(w + s_w0[i])) : 0.f;
            s_a[buf][tt][i] = fa[n];
            s_k[buf][tt][i] = fk[n];
            s_w[buf][tt][i] = w;
        }
#pragma unroll
        for (int n = 0; n < V_ITEMS; ++n) {
            const int idx = n * THREADS + threadIdx.x;
            if (idx < CHUNK * CTA_COLS) s_v[buf][idx / CTA_COLS][idx % CTA_COLS] = fv[n];
        }
        if (RULE == 0 && threadIdx.x < CHUNK) s_beta[buf][threadIdx.x] = fb;
    };

    fetch(first);
    __syncthreads();            // s_w0 is there
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int c0 = first; c0 < len; c0 += CHUNK, buf ^= 1) {
        const int nt = min(CHUNK, len - c0);
        const bool more = c0 + CHUNK < len;
        if (more) fetch(c0 + CHUNK);
        for (int tt = 0; tt < nt; ++tt) {
            const float4* w4 = reinterpret_cast<const float4*>(&s_w[buf][tt][4 * il]);
            const float4* k4 = reinterpret_cast<const float4*>(&s_k[buf][tt][4 * il]);
            const float4* a4 = reinterpret_cast<const float4*>(&s_a[buf][tt][4 * il]);
            float vj[NC], out[NC];
#pragma unroll
            for (int c = 0; c < NC; ++c) vj[c] = s_v[buf][tt][jc + c * COLS];
            // four partial sums a read (fixed order): a single chain of R dependent additions would set the pace
            if (RULE == 0) {
                float d[NC][4], kk[R];
#pragma unroll
                for (int c = 0; c < NC; ++c) d[c][0] = d[c][1] = d[c][2] = d[c][3] = 0.f;
#pragma unroll
                for (int g = 0; g < R / 4; ++g) {
                    const float4 w = w4[LANES * g], k = k4[LANES * g];
                    const float wv[4] = {w.x, w.y, w.z, w.w};
                    kk[4 * g] = k.x; kk[4 * g + 1] = k.y; kk[4 * g + 2] = k.z; kk[4 * g + 3] = k.w;
#pragma unroll
                    for (int c = 0; c < NC; ++c)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            S[c][4 * g + e] = fmaf(S[c][4 * g + e], wv[e], S[c][4 * g + e]);
                            d[c][e] = fmaf(S[c][4 * g + e], kk[4 * g + e], d[c][e]);
                        }
                }
                float u[NC];
#pragma unroll
                for (int c = 0; c < NC; ++c) u[c] = (d[c][0] + d[c][1]) + (d[c][2] + d[c][3]);
#pragma unroll
                for (int o = 1; o < LANES; o <<= 1)
#pragma unroll
                    for (int c = 0; c < NC; ++c) u[c] += __shfl_xor_sync(0xffffffffu, u[c], o);
                const float beta = s_beta[buf][tt];
#pragma unroll
                for (int c = 0; c < NC; ++c) u[c] = beta * (vj[c] - u[c]);
                float acc[NC][4];
#pragma unroll
                for (int c = 0; c < NC; ++c) acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
#pragma unroll
                for (int g = 0; g < R / 4; ++g) {
                    const float4 q = a4[LANES * g];
                    const float qv[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int c = 0; c < NC; ++c)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            S[c][4 * g + e] = fmaf(kk[4 * g + e], u[c], S[c][4 * g + e]);
                            acc[c][e] = fmaf(S[c][4 * g + e], qv[e], acc[c][e]);
                        }
                }
#pragma unroll
                for (int c = 0; c < NC; ++c) out[c] = (acc[c][0] + acc[c][1]) + (acc[c][2] + acc[c][3]);
            } else {
                const float4* b4 = reinterpret_cast<const float4*>(&s_bonus[4 * il]);
                float acc[NC][4];
#pragma unroll
                for (int c = 0; c < NC; ++c) acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
#pragma unroll
                for (int g = 0; g < R / 4; ++g) {
                    const float4 w = w4[LANES * g], k = k4[LANES * g], rr = a4[LANES * g], b = b4[LANES * g];
                    const float wv[4] = {w.x, w.y, w.z, w.w}, kv4[4] = {k.x, k.y, k.z, k.w}, rv[4] = {rr.x, rr.y, rr.z, rr.w},
                                bv[4] = {b.x, b.y, b.z, b.w};
                    if (mode == 1) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) decayed[4 * g + e] = fmaf(wv[e], decayed[4 * g + e], decayed[4 * g + e]);
                    }
#pragma unroll
                    for (int c = 0; c < NC; ++c)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float kv = kv4[e] * vj[c];
                            acc[c][e] = fmaf(rv[e], fmaf(bv[e], kv, S[c][4 * g + e]), acc[c][e]);
                            S[c][4 * g + e] = fmaf(wv[e], S[c][4 * g + e], S[c][4 * g + e]) + kv;
                        }
                }
#pragma unroll
                for (int c = 0; c < NC; ++c) out[c] = (acc[c][0] + acc[c][1]) + (acc[c][2] + acc[c][3]);
            }
#pragma unroll
            for (int o = 1; o < LANES; o <<= 1)
#pragma unroll
                for (int c = 0; c < NC; ++c) out[c] += __shfl_xor_sync(0xffffffffu, out[c], o);
            if (il == 0 && mode != 1) {
#pragma unroll
                for (int c = 0; c < NC; ++c)
                    if (j0 + c * COLS < DV) p.o[(static_cast<size_t>(start + c0 + tt) * H + h) * DV + j0 + c * COLS] = out[c];
            }
        }
        if (more) stash(buf ^ 1);       // nobody reads that buffer: its chunk was finished before the last barrier
        __syncthreads();
    }
    if (mode != 2) {
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = row_of(r), j = j0 + c * COLS;
                if (i < D && j < DV) S_g[static_cast<size_t>(i) * DV + j] = S[c][r];
            }
    }
    if (mode == 1) {
        if (RULE == 1 && blockIdx.x == 0 && jc == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r)
                if (row_of(r) < D) p.piece_p[(static_cast<size_t>(blockIdx.z) * H + h) * D + row_of(r)] = decayed[r];
        }
        return;
    }
    if (mode == 2 && first != 0) return;          // the CTAs of a request's first piece move the tail
    // The convolution's tail: row m of the new tail is the input of local token len - (taps - 1) + m, which lies in
    // this step or, for a short step, further up in the old tail. Channels are shared out over the CTAs of the request;
    // a channel's rows move in ascending order, so a row is read before it is overwritten.
    if (p.taps > 1) {
        const int keep = p.taps - 1;
        const int all = PIECES ? p.q_len[seq] : len;        // the whole request's tokens, whatever this CTA's piece
        float* tail = p.state + static_cast<size_t>(p.state_slot[seq]) * p.state_stride + p.tail_off;
        const int cta = blockIdx.y * gridDim.x + blockIdx.x, ctas = gridDim.x * gridDim.y;
        for (int c = cta * blockDim.x + threadIdx.x; c < p.C; c += ctas * blockDim.x)
            for (int m = 0; m < keep; ++m) {
                const int src = all - keep + m;
                tail[static_cast<size_t>(m) * p.C + c] = src >= 0 ? load_any(p.proj, static_cast<size_t>(start + src) * p.ld_proj + c, p.proj_bf16)
                                                                 : tail[static_cast<size_t>(m + all) * p.C + c];
            }
    }
}

// Between the two passes over pieces, for a memory whose decay is diagonal: piece_s [z, H, D, DV] holds what every piece
// adds from a zero memory, piece_p [z, H, D] the product of its decays. One thread an entry of S walks the request's pieces
// in order: the memory at a piece's start takes the place of the piece's own sum, and the memory after the last piece goes
// into the state.
__global__ void __launch_bounds__(256)
pieces_combine_kernel(float* __restrict__ piece_s, const float* __restrict__ piece_p, float* __restrict__ state, long long state_stride,
                      const int32_t* __restrict__ q_len, const int32_t* __restrict__ state_slot, int H, int D, int DV, int piece,
                      int max_pieces) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.y;
    const int len = q_len[seq];
    if (len <= 0) return;
    const int entry = blockIdx.x * blockDim.x + threadIdx.x;          // over H * D * DV
    if (entry >= H * D * DV) return;
    const int row = entry / DV;                                          // h * D + i
    float* S_g = state + static_cast<size_t>(state_slot[seq]) * state_stride + entry;
    float S = *S_g;
    const int pieces = (len + piece - 1) / piece;
    for (int c = 0; c < pieces; ++c) {
        const size_t z = static_cast<size_t>(seq) * max_pieces + c;
        float* at = piece_s + z * H * D * DV + entry;
        const float own = *at;
        *at = S;
        S = fmaf(piece_p[z * H * D + row], S, own);
    }
    *S_g = S;
}

// The same for the delta rule, whose pieces carry a memory across by a full matrix: piece_t [z, H, D, D] holds it, piece_s
// [z, H, D, DV] what the piece adds from a zero memory; S_next = T S + B. A CTA owns 16 columns of S of one head of one
// request and walks the pieces in order; T comes through shared memory in slabs of 16 columns. The memory at a piece's
// start takes the place of the piece's own sum, the memory after the last piece goes into the state.
constexpr int kCombineCols = 16, kCombineThreads = 256, kCombineMaxD = 256;

__global__ void __launch_bounds__(kCombineThreads)
delta_pieces_combine_kernel(float* __restrict__ piece_s, const float* __restrict__ piece_t, float* __restrict__ state,
                            long long state_stride, const int32_t* __restrict__ q_len, const int32_t* __restrict__ state_slot, int H, int D,
                            int DV, int piece, int max_pieces) {
    pdl_trigger();
    pdl_wait();
    constexpr int PER = kCombineMaxD * kCombineCols / kCombineThreads;       // entries of the CTA's columns a thread, at most
    __shared__ float S_s[kCombineMaxD][kCombineCols], T_s[kCombineMaxD][kCombineCols + 1];
    const int seq = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * kCombineCols;
    const int len = q_len[seq];
    if (len <= 0) return;
    float* S_g = state + static_cast<size_t>(state_slot[seq]) * state_stride + static_cast<size_t>(h) * D * DV;
    const int entries = D * kCombineCols;
    for (int idx = threadIdx.x; idx < entries; idx += kCombineThreads) {
        const int row = idx / kCombineCols, col = idx % kCombineCols;
        S_s[row][col] = c0 + col < DV ? S_g[static_cast<size_t>(row) * DV + c0 + col] : 0.f;
    }
    __syncthreads();
    const int pieces = (len + piece - 1) / piece;
    for (int c = 0; c < pieces; ++c) {
        const size_t z = static_cast<size_t>(seq) * max_pieces + c;
        const float* T = piece_t + (z * H + h) * D * D;
        float* B = piece_s + (z * H + h) * D * DV;
        float acc[PER];
#pragma unroll
        for (int n = 0; n < PER; ++n) acc[n] = 0.f;
        for (int k0 = 0; k0 < D; k0 += kCombineCols) {
            for (int idx = threadIdx.x; idx < entries; idx += kCombineThreads) {
                const int row = idx / kCombineCols, kk = idx % kCombineCols;
                T_s[row][kk] = k0 + kk < D ? T[static_cast<size_t>(row) * D + k0 + kk] : 0.f;
            }
            __syncthreads();
#pragma unroll
            for (int n = 0; n < PER; ++n) {
                const int idx = n * kCombineThreads + threadIdx.x;
                if (idx < entries) {
                    const int row = idx / kCombineCols, col = idx % kCombineCols;
#pragma unroll
                    for (int kk = 0; kk < kCombineCols; ++kk)
                        if (k0 + kk < D) acc[n] = fmaf(T_s[row][kk], S_s[k0 + kk][col], acc[n]);
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int n = 0; n < PER; ++n) {
            const int idx = n * kCombineThreads + threadIdx.x;
            if (idx < entries) {
                const int row = idx / kCombineCols, col = idx % kCombineCols;
                if (c0 + col < DV) {
                    float* at = B + static_cast<size_t>(row) * DV + c0 + col;
                    const float own = *at;
                    *at = S_s[row][col];                // every thread reads and writes its own entries only
                    acc[n] += own;
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int n = 0; n < PER; ++n) {
            const int idx = n * kCombineThreads + threadIdx.x;
            if (idx < entries) S_s[idx / kCombineCols][idx % kCombineCols] = acc[n];
        }
        __syncthreads();
    }
    for (int idx = threadIdx.x; idx < entries; idx += kCombineThreads) {
        const int row = idx / kCombineCols, col = idx % kCombineCols;
        if (c0 + col < DV) S_g[static_cast<size_t>(row) * DV + c0 + col] = S_s[row][col];
    }
}

template <int LANES, int R, int CHUNK, int RULE>
int launch_scan_as(const ScanArgs& p, int num_seqs, cudaStream_t stream) {
    constexpr int COLS = kScanThreads / LANES;
    // four columns a thread where the head is wide enough to fill them
    if (p.mode) num_seqs *= p.max_pieces;
    if (p.DV >= 4 * COLS) {
        const dim3 grid((p.DV + 4 * COLS - 1) / (4 * COLS), p.H, num_seqs);
        if (p.mode) stride::launch_alone(scan_kernel<LANES, R, 4, CHUNK, RULE, true>, grid, dim3(kScanThreads), 0, stream, p);
        else stride::launch_alone(scan_kernel<LANES, R, 4, CHUNK, RULE, false>, grid, dim3(kScanThreads), 0, stream, p);
    } else {
        const dim3 grid((p.DV + COLS - 1) / COLS, p.H, num_seqs);
        if (p.mode) stride::launch_alone(scan_kernel<LANES, R, 1, CHUNK, RULE, true>, grid, dim3(kScanThreads), 0, stream, p);
        else stride::launch_alone(scan_kernel<LANES, R, 1, CHUNK, RULE, false>, grid, dim3(kScanThreads), 0, stream, p);
    }
    return STRIDE_LAUNCH_STATUS();
}

template <int RULE>
int launch_scan(const ScanArgs& p, int num_seqs, cudaStream_t stream) {
    if (p.D <= 16) return launch_scan_as<4, 4, 16, RULE>(p, num_seqs, stream);
    if (p.D <= 32) return launch_scan_as<8, 4, 16, RULE>(p, num_seqs, stream);
    if (p.D <= 64) return launch_scan_as<16, 4, 16, RULE>(p, num_seqs, stream);
    if (p.D <= 128) return launch_scan_as<16, 8, 8, RULE>(p, num_seqs, stream);
    if (p.D <= 256) return launch_scan_as<16, 16, 4, RULE>(p, num_seqs, stream);
    return STRIDE_UNSUPPORTED;
}

}  // namespace stride

using namespace stride;

extern "C" {

int stride_delta_prepare(const void* proj, int ld, const float* conv_w, const float* low, int ld_low, const float* a_log,
                         const float* dt_bias, const float* state, long long state_stride, long long tail_off,
                         const int32_t* seq_of_token, const int32_t* q_start, const int32_t* state_slot, float* qk, float* v_out,
                         float* beta, float* decay, int tokens, int G, int H, int D, int DV, int taps, float unit_eps, int dtype,
                         cudaStream_t stream) {
    if (tokens < 0 || G <= 0 || H <= 0 || D <= 0 || DV <= 0 || taps <= 0 || H % G) return STRIDE_BAD_ARGUMENT;
    if (D > 32 * kMaxPerLane || DV > 32 * kMaxPerLane) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    const dim3 grid(tokens, (2 * G + H + kPrepWarps - 1) / kPrepWarps), block(kPrepWarps * 32);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(delta_prepare_kernel<float>, grid, block, 0, stream, static_cast<const float*>(proj), ld, conv_w, low, ld_low, a_log,
                       dt_bias, state, state_stride, tail_off, seq_of_token, q_start, state_slot, qk, v_out, beta, decay, G, H, D, DV, taps,
                       unit_eps);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(delta_prepare_kernel<__nv_bfloat16>, grid, block, 0, stream, static_cast<const __nv_bfloat16*>(proj), ld, conv_w, low,
                       ld_low, a_log, dt_bias, state, state_stride, tail_off, seq_of_token, q_start, state_slot, qk, v_out, beta, decay, G, H,
                       D, DV, taps, unit_eps);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

// The gated delta rule over the step's requests. qk, v, beta, decay: what delta_prepare wrote. proj: the projections
// whose last taps - 1 rows become the convolution's new tail.
// piece > 0: in pieces of that many tokens, parallel over the pieces (every piece from a zero memory; every piece's matrix;
// the memories at the pieces' starts; every piece from its start). scratch: float32, at least
// num_seqs * max_pieces * H * D * (DV + D). As for the other rule, the sums then take another order than the chain's.
int stride_delta_scan(const float* qk, const float* v, const float* beta, const float* decay, float* o, float* state,
                      long long state_stride, long long tail_off, const void* proj, int ld_proj, const int32_t* q_start,
                      const int32_t* q_len, const int32_t* state_slot, int num_seqs, int G, int H, int D, int DV, int taps, int dtype,
                      int piece, int max_pieces, float* scratch, cudaStream_t stream) {
    if (num_seqs < 0 || G <= 0 || H <= 0 || D <= 0 || DV <= 0 || taps <= 0 || H % G) return STRIDE_BAD_ARGUMENT;
    if (piece < 0 || (piece > 0 && (max_pieces <= 0 || scratch == nullptr))) return STRIDE_BAD_ARGUMENT;
    if (piece > 0 && D > kCombineMaxD) return STRIDE_UNSUPPORTED;
    if (dtype != STRIDE_DTYPE_F32 && dtype != STRIDE_DTYPE_BF16) return STRIDE_BAD_ARGUMENT;
    if (num_seqs == 0) return 0;
    ScanArgs p = {};
    p.a = qk;
    p.k = qk + static_cast<size_t>(G) * D;
    p.lda = 2 * G * D;
    p.w = decay;
    p.v = v;
    p.ldv = H * DV;
    p.beta = beta;
    p.o = o;
    p.state = state;
    p.state_stride = state_stride;
    p.q_start = q_start;
    p.q_len = q_len;
    p.state_slot = state_slot;
    p.H = H;
    p.group = H / G;
    p.D = D;
    p.DV = DV;
    p.in_bf16 = 0;
    p.proj = proj;
    p.ld_proj = ld_proj;
    p.C = 2 * G * D + H * DV;
    p.taps = taps;
    p.tail_off = tail_off;
    p.proj_bf16 = dtype == STRIDE_DTYPE_BF16 ? 1 : 0;      // the tail is read in the projections' type, the rest is float32
    if (piece == 0) return launch_scan<0>(p, num_seqs, stream);
    const size_t zs = static_cast<size_t>(num_seqs) * max_pieces;
    float* piece_s = scratch;
    float* piece_t = scratch + zs * H * D * DV;
    p.piece = piece;
    p.max_pieces = max_pieces;
    p.mode = 1;
    p.init = 1;
    p.piece_s = piece_s;
    int code = launch_scan<0>(p, num_seqs, stream);             // what every piece adds from a zero memory
    if (code != 0) return code;
    ScanArgs t = p;
    t.v = nullptr;
    t.DV = D;
    t.init = 2;
    t.piece_s = piece_t;
    code = launch_scan<0>(t, num_seqs, stream);                 // every piece's matrix
    if (code != 0) return code;
    stride::launch(delta_pieces_combine_kernel, dim3((DV + kCombineCols - 1) / kCombineCols, H, num_seqs), dim3(kCombineThreads), 0, stream,
                   piece_s, static_cast<const float*>(piece_t), state, state_stride, q_len, state_slot, H, D, DV, piece, max_pieces);
    code = STRIDE_LAUNCH_STATUS();
    if (code != 0) return code;
    p.mode = 2;
    return launch_scan<0>(p, num_seqs, stream);                 // every piece from its start, with the outputs
}

// Decayed memory with a bonus. r, k, v [tokens, H * D] in the compute type (one head size for keys and values);
// wlog [tokens, H * D] float32: the decay is exp(-exp(wlog + w0)).
// piece > 0: the recurrence in pieces of that many tokens, parallel over the pieces (three launches: every piece from a zero
// memory; the memories at the pieces' starts; every piece from its start). scratch: float32, at least
// num_seqs * max_pieces * H * D * (D + 1), max_pieces = ceil(longest portion / piece). The sums then take another order than
// the single chain's, so the result depends on the cutting in the last bits: for bfloat16 runs and long portions.
int stride_bonus_scan(const void* r, const void* k, const void* v, const float* wlog, const float* w0, const float* bonus, float* o,
                      float* state, long long state_stride, const int32_t* q_start, const int32_t* q_len, const int32_t* state_slot,
                      int num_seqs, int H, int D, int dtype, int piece, int max_pieces, float* scratch, cudaStream_t stream) {
    if (num_seqs < 0 || H <= 0 || D <= 0 || piece < 0 || (piece > 0 && (max_pieces <= 0 || scratch == nullptr))) return STRIDE_BAD_ARGUMENT;
    if (dtype != STRIDE_DTYPE_F32 && dtype != STRIDE_DTYPE_BF16) return STRIDE_BAD_ARGUMENT;
    if (num_seqs == 0) return 0;
    ScanArgs p = {};
    p.a = r;
    p.k = k;
    p.lda = H * D;
    p.w = wlog;
    p.w0 = w0;
    p.bonus = bonus;
    p.v = v;
    p.ldv = H * D;
    p.o = o;
    p.state = state;
    p.state_stride = state_stride;
    p.q_start = q_start;
    p.q_len = q_len;
    p.state_slot = state_slot;
    p.H = H;
    p.group = 1;
    p.D = D;
    p.DV = D;
    p.in_bf16 = dtype == STRIDE_DTYPE_BF16 ? 1 : 0;
    p.taps = 0;
    if (piece == 0) return launch_scan<1>(p, num_seqs, stream);
    p.piece = piece;
    p.max_pieces = max_pieces;
    p.piece_s = scratch;
    p.piece_p = scratch + static_cast<size_t>(num_seqs) * max_pieces * H * D * D;
    p.mode = 1;
    int code = launch_scan<1>(p, num_seqs, stream);
    if (code != 0) return code;
    const int entries = H * D * D;
    stride::launch(pieces_combine_kernel, dim3((entries + 255) / 256, num_seqs), dim3(256), 0, stream, p.piece_s,
                   static_cast<const float*>(p.piece_p), state, state_stride, q_len, state_slot, H, D, D, piece, max_pieces);
    code = STRIDE_LAUNCH_STATUS();
    if (code != 0) return code;
    p.mode = 2;
    return launch_scan<1>(p, num_seqs, stream);
}

int stride_shift_mix(const void* x, const float* mu, float* state, long long state_stride, long long prev_off,
                     const int32_t* seq_of_token, const int32_t* q_start, const int32_t* q_len, const int32_t* state_slot, void* out,
                     int tokens, int width, int mixes, int dtype, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || mixes <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(shift_mix_kernel<float>, dim3(tokens), dim3(256), 0, stream, static_cast<const float*>(x), mu, state, state_stride,
                       prev_off, seq_of_token, q_start, q_len, state_slot, static_cast<float*>(out), tokens, width, mixes);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(shift_mix_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), mu, state,
                       state_stride, prev_off, seq_of_token, q_start, q_len, state_slot, static_cast<__nv_bfloat16*>(out), tokens, width,
                       mixes);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_head_norm_gate(const float* o, const float* weight, int w_head_stride, const void* gate, int ld_gate, int gate_kind, void* out,
                          int tokens, int H, int DV, float eps, int dtype, cudaStream_t stream) {
    if (tokens < 0 || H <= 0 || DV <= 0 || gate_kind < 0 || gate_kind > 2) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const long long pairs = static_cast<long long>(tokens) * H;
    const dim3 grid(static_cast<unsigned>((pairs + 7) / 8)), block(256);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(head_norm_gate_kernel<float>, grid, block, 0, stream, o, weight, w_head_stride, gate, ld_gate, gate_kind,
                       static_cast<float*>(out), tokens, H, DV, eps);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(head_norm_gate_kernel<__nv_bfloat16>, grid, block, 0, stream, o, weight, w_head_stride, gate, ld_gate, gate_kind,
                       static_cast<__nv_bfloat16*>(out), tokens, H, DV, eps);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
