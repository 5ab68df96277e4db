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
// column the only coupling is the sum over D of a read. A column belongs to 8 neighbouring lanes, lane l holding rows l,
// l + 8, ... in registers together with the same rows of n (every column's lanes keep n for themselves: D / 8 more
// multiply-adds a token, and no exchange between columns). A CTA of 128 threads owns 16 columns of one head of one request and
// walks the request's tokens of the step in order; the inputs of 16 tokens are staged in shared memory at a time (q already
// times `q_scale`, the two gate logarithms computed once a token). Every thread follows the chain of m itself: its
// exponentials do not depend on the memory and run beside the sums. The order of every sum depends on the token only, so a
// token's output is bitwise the same in a whole prompt, in portions or decoded alone.
//
// State row of a request: S [H, D, DV], then n [H, D], then m [H].
#include "common.cuh"

namespace stride {

constexpr int kLstmThreads = 128;
constexpr int kLstmLanes = 8;
constexpr int kLstmCols = kLstmThreads / kLstmLanes;
constexpr int kLstmChunk = 16;

struct LstmArgs {
    const void* proj;       // [tokens, ld] in the compute type: q of head h at q_off + h * D, k at k_off + h * D, v at v_off + h * DV
    int ld, q_off, k_off, v_off, is_bf16;
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

__device__ __forceinline__ float lstm_load(const void* p, size_t i, int is_bf16) {
    return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]) : static_cast<const float*>(p)[i];
}

__device__ __forceinline__ float log_sigmoid_f(float z) { return z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z)); }

template <int R>
__global__ void __launch_bounds__(kLstmThreads)
mlstm_scan_kernel(const LstmArgs p) {
    constexpr int DP = R * kLstmLanes;
    __shared__ float s_q[kLstmChunk][DP], s_k[kLstmChunk][DP];
    __shared__ float s_v[kLstmChunk][kLstmCols], s_li[kLstmChunk], s_lf[kLstmChunk];
    const int seq = blockIdx.z, h = blockIdx.y;
    const int len = p.q_len[seq];
    if (len <= 0) return;
    const int start = p.q_start[seq];
    const int il = threadIdx.x & (kLstmLanes - 1), jc = threadIdx.x / kLstmLanes;
    const int j = blockIdx.x * kLstmCols + jc;
    const int H = p.H, D = p.D, DV = p.DV;
    float* base = p.state + static_cast<size_t>(p.state_slot[seq]) * p.state_stride;
    float* S_g = base + static_cast<size_t>(h) * D * DV;
    float* n_g = base + static_cast<size_t>(H) * D * DV + static_cast<size_t>(h) * D;
    float* m_g = base + static_cast<size_t>(H) * D * DV + static_cast<size_t>(H) * D + h;
    float S[R], nn[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = il + kLstmLanes * r;
        S[r] = (i < D && j < DV) ? S_g[static_cast<size_t>(i) * DV + j] : 0.f;
        nn[r] = i < D ? n_g[i] : 0.f;
    }
    float m = *m_g;
    for (int c0 = 0; c0 < len; c0 += kLstmChunk) {
        const int nt = min(kLstmChunk, len - c0);
        __syncthreads();            // the chunk before has been read by everybody
        for (int idx = threadIdx.x; idx < kLstmChunk * DP; idx += kLstmThreads) {
            const int tt = idx / DP, i = idx - tt * DP;
            float q = 0.f, k = 0.f;
            if (tt < nt && i < D) {
                const size_t row = static_cast<size_t>(start + c0 + tt) * p.ld;
                q = lstm_load(p.proj, row + p.q_off + h * D + i, p.is_bf16) * p.q_scale;
                k = lstm_load(p.proj, row + p.k_off + h * D + i, p.is_bf16);
            }
            s_q[tt][i] = q;
            s_k[tt][i] = k;
        }
        for (int idx = threadIdx.x; idx < kLstmChunk * kLstmCols; idx += kLstmThreads) {
            const int tt = idx / kLstmCols, c = idx - tt * kLstmCols;
            const int col = blockIdx.x * kLstmCols + c;
            s_v[tt][c] = (tt < nt && col < DV) ? lstm_load(p.proj, static_cast<size_t>(start + c0 + tt) * p.ld + p.v_off + h * DV + col, p.is_bf16)
                                                : 0.f;
        }
        if (threadIdx.x < nt) {
            const size_t row = static_cast<size_t>(start + c0 + threadIdx.x) * p.ld_gates;
            const float zi = p.gates[row + h] + p.bias_i[h], zf = p.gates[row + H + h] + p.bias_f[h];
            s_li[threadIdx.x] = p.cap * tanhf(zi / p.cap);
            s_lf[threadIdx.x] = log_sigmoid_f(p.cap * tanhf(zf / p.cap));
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float li = s_li[tt], lf = s_lf[tt];
            const float m_new = fmaxf(lf + m, li);
            const float keep = expf(lf + m - m_new), take = expf(li - m_new), floor_ = expf(-m_new);
            m = m_new;
            const float vj = s_v[tt][jc] * take;
            float acc[4] = {0.f, 0.f, 0.f, 0.f}, den[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float kk = s_k[tt][il + kLstmLanes * r], qq = s_q[tt][il + kLstmLanes * r];
                S[r] = fmaf(keep, S[r], kk * vj);
                nn[r] = fmaf(keep, nn[r], take * kk);
                acc[r & 3] = fmaf(S[r], qq, acc[r & 3]);
                den[r & 3] = fmaf(nn[r], qq, den[r & 3]);
            }
            float num = (acc[0] + acc[1]) + (acc[2] + acc[3]), dot = (den[0] + den[1]) + (den[2] + den[3]);
#pragma unroll
            for (int o = 1; o < kLstmLanes; o <<= 1) {
                num += __shfl_xor_sync(0xffffffffu, num, o);
                dot += __shfl_xor_sync(0xffffffffu, dot, o);
            }
            if (il == 0 && j < DV)
                p.o[(static_cast<size_t>(start + c0 + tt) * H + h) * DV + j] = num / (fmaxf(fabsf(dot), floor_) + 1e-6f);
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = il + kLstmLanes * r;
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
    a.proj = proj; a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.is_bf16 = dtype == STRIDE_DTYPE_BF16;
    a.gates = gates; a.ld_gates = ld_gates; a.bias_i = bias_i; a.bias_f = bias_f; a.cap = cap; a.q_scale = q_scale;
    a.o = o; a.state = state; a.state_stride = state_stride; a.q_start = q_start; a.q_len = q_len; a.state_slot = state_slot;
    a.H = H; a.D = D; a.DV = DV;
    const dim3 grid((DV + kLstmCols - 1) / kLstmCols, H, num_seqs), block(kLstmThreads);
    const int rows = (D + kLstmLanes - 1) / kLstmLanes;
    // a chain of tokens keeps few CTAs busy for long: launched without an early start behind the kernel before it
    if (rows <= 2) stride::launch_alone(mlstm_scan_kernel<2>, grid, block, 0, stream, a);
    else if (rows <= 4) stride::launch_alone(mlstm_scan_kernel<4>, grid, block, 0, stream, a);
    else if (rows <= 8) stride::launch_alone(mlstm_scan_kernel<8>, grid, block, 0, stream, a);
    else if (rows <= 16) stride::launch_alone(mlstm_scan_kernel<16>, grid, block, 0, stream, a);
    else stride::launch_alone(mlstm_scan_kernel<32>, grid, block, 0, stream, a);
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
