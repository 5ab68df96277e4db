// A short causal convolution over time on every channel of the fused q/k/v projection, followed by what attention needs of
// its result: RMS norms per query and key head with a weight shared by the heads, and the write of keys and values into
// their pages.
//
//   conv_head_norm   raw [tokens, ld]: columns [q heads | k heads | v heads] as projected. For channel c of token t
//                      y_t[c] = sum_j w[j, c] * u_(t - taps + 1 + j)[c]          (w [taps, C]: a tap's weights side by side)
//                    where u is the projected value of the same request: a row of this step, or, before the step's first
//                    token, a row of the request's tail (the last taps - 1 projected rows, float32, in the request's state
//                    slot; zeros for a request that starts). Then y / sqrt(mean(y^2) + eps) * weight per query and key
//                    head (a null weight leaves the head as it is), the result into `out` (same column layout) and keys
//                    and values into the pages [page, kv_head, slot, width]. A null w: no convolution; taps 1: one factor
//                    a channel.
//   conv_tail        afterwards, the tails move on: row m of the new tail is the projected row of local token
//                    len - (taps - 1) + m, which lies in this step or, for a short step, further up in the old tail.
//                    A thread owns a channel and reads all it needs before it writes.
// One warp a (token, head); float32 arithmetic; sums in an order that depends on the head's width only. Heads of whole
// 16-byte packs on 16-byte boundaries take the packed form: a lane holds whole packs of its head (8 bfloat16 or 4 float32
// channels), a warp serves one head of up to 32 packs or two heads of up to 16, and every row of a tap is one 16-byte read.
#include "common.cuh"

namespace stride {

constexpr int kConvWarps = 4;
constexpr int kConvMaxHead = 256;
constexpr int kConvMaxTaps = 16;

template <typename T>
__global__ void __launch_bounds__(kConvWarps * 32)
conv_head_norm_kernel(const T* __restrict__ raw, int ld, T* __restrict__ out, int ld_out, const float* __restrict__ conv_w, int taps,
                      const float* __restrict__ state, long long state_stride, long long tail_off,
                      const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ q_start,
                      const int32_t* __restrict__ state_slot, const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                      const int32_t* __restrict__ slot_mapping, T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv, int hd,
                      int vd, int page_size) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * kConvWarps + warp;          // query heads, then key heads, then value heads
    if (head >= nq + 2 * nkv) return;
    const int seq = seq_of_token[t];
    if (seq < 0) return;
    const bool is_value = head >= nq + nkv;
    const int width = is_value ? vd : hd;
    const int column = is_value ? (nq + nkv) * hd + (head - nq - nkv) * vd : head * hd;
    const int C = (nq + nkv) * hd + nkv * vd;
    const int start = q_start[seq];
    const int local = t - start;
    const float* tail = state ? state + static_cast<size_t>(state_slot[seq]) * state_stride + tail_off : nullptr;
    float v[kConvMaxHead / 32];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < kConvMaxHead / 32; ++i) {
        const int d = lane + 32 * i;
        v[i] = 0.f;
        if (d < width) {
            const int c = column + d;
            if (conv_w && taps > 1) {
                float acc = 0.f;
                for (int j = 0; j < taps; ++j) {
                    const int src = local - (taps - 1) + j;
                    const float u = src >= 0 ? to_f32(raw[static_cast<size_t>(start + src) * ld + c])
                                             : tail[static_cast<size_t>(taps - 1 + src) * C + c];
                    acc = fmaf(conv_w[static_cast<size_t>(j) * C + c], u, acc);
                }
                v[i] = acc;
            } else {
                v[i] = to_f32(raw[static_cast<size_t>(t) * ld + c]);
                if (conv_w) v[i] *= conv_w[c];
            }
            sq = fmaf(v[i], v[i], sq);
        }
    }
    const float* weight = is_value ? nullptr : (head < nq ? wq : wk);
    const float inv = weight ? rsqrtf(warp_sum(sq) / static_cast<float>(width) + eps) : 1.f;
    const int slot = (slot_mapping && head >= nq) ? slot_mapping[t] : -1;
    T* dst = nullptr;
    if (slot >= 0) {
        const int kvh = is_value ? head - nq - nkv : head - nq;
        dst = (is_value ? v_pages : k_pages) + ((static_cast<size_t>(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * width;
    }
    T* x = out + static_cast<size_t>(t) * ld_out + column;
#pragma unroll
    for (int i = 0; i < kConvMaxHead / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < width) {
            const T y = from_f32<T>(weight ? __fmul_rn(__fmul_rn(v[i], inv), weight[d]) : v[i]);
            x[d] = y;
            if (dst) dst[d] = y;
        }
    }
}

template <typename T>
struct ConvPack;
template <>
struct ConvPack<float> {
    static constexpr int V = 4;
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <>
struct ConvPack<__nv_bfloat16> {
    static constexpr int V = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
        const uint4 r = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        uint4 r;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        *reinterpret_cast<uint4*>(p) = r;
    }
};

// The packed form. LANES = 32: one head a warp; LANES = 16: two heads a warp, for heads of at most 16 packs (the sum of a
// head then stays inside a half warp). A channel's taps are summed in the order of the plain form.
template <typename T, int LANES>
__global__ void __launch_bounds__(kConvWarps * 32)
conv_head_norm_vec_kernel(const T* __restrict__ raw, int ld, T* __restrict__ out, int ld_out, const float* __restrict__ conv_w, int taps,
                          const float* __restrict__ state, long long state_stride, long long tail_off,
                          const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ q_start,
                          const int32_t* __restrict__ state_slot, const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                          const int32_t* __restrict__ slot_mapping, T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv,
                          int hd, int vd, int page_size) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = ConvPack<T>::V;
    constexpr int kPacks = LANES == 32 ? kConvMaxHead / (32 * V) : 1;
    constexpr int kPerWarp = 32 / LANES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & (LANES - 1);
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0) return;
    const int head = (blockIdx.y * kConvWarps + warp) * kPerWarp + ((threadIdx.x & 31) / LANES);
    const bool live = head < nq + 2 * nkv;        // a half warp without a head still takes part in the shuffles
    const bool is_value = head >= nq + nkv;
    const int width = live ? (is_value ? vd : hd) : 0;
    const int column = live ? (is_value ? (nq + nkv) * hd + (head - nq - nkv) * vd : head * hd) : 0;
    const int C = (nq + nkv) * hd + nkv * vd;
    const int start = q_start[seq];
    const int local = t - start;
    const float* tail = state ? state + static_cast<size_t>(state_slot[seq]) * state_stride + tail_off : nullptr;
    float v[kPacks][V];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < kPacks; ++i) {
        const int d = (lane + LANES * i) * V;
        if (d < width) {
            const int c = column + d;
            if (conv_w && taps > 1) {
#pragma unroll
                for (int e = 0; e < V; ++e) v[i][e] = 0.f;
                for (int j = 0; j < taps; ++j) {
                    const int src = local - (taps - 1) + j;
                    float u[V];
                    if (src >= 0) {
                        ConvPack<T>::load(raw + static_cast<size_t>(start + src) * ld + c, u);
                    } else {
                        const float* row = tail + static_cast<size_t>(taps - 1 + src) * C + c;
#pragma unroll
                        for (int e = 0; e < V; e += 4) ConvPack<float>::load(row + e, u + e);
                    }
                    float w[V];
#pragma unroll
                    for (int e = 0; e < V; e += 4) ConvPack<float>::load(conv_w + static_cast<size_t>(j) * C + c + e, w + e);
#pragma unroll
                    for (int e = 0; e < V; ++e) v[i][e] = fmaf(w[e], u[e], v[i][e]);
                }
            } else {
                ConvPack<T>::load(raw + static_cast<size_t>(t) * ld + c, v[i]);
                if (conv_w) {
#pragma unroll
                    for (int e = 0; e < V; ++e) v[i][e] *= conv_w[c + e];
                }
            }
#pragma unroll
            for (int e = 0; e < V; ++e) sq = fmaf(v[i][e], v[i][e], sq);
        }
    }
    const float* weight = (!live || is_value) ? nullptr : (head < nq ? wq : wk);
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float inv = weight ? rsqrtf(sq / static_cast<float>(width) + eps) : 1.f;
    const int slot = (slot_mapping && live && head >= nq) ? slot_mapping[t] : -1;
    T* dst = nullptr;
    if (slot >= 0) {
        const int kvh = is_value ? head - nq - nkv : head - nq;
        dst = (is_value ? v_pages : k_pages) + ((static_cast<size_t>(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * width;
    }
    T* x = out + static_cast<size_t>(t) * ld_out + column;
#pragma unroll
    for (int i = 0; i < kPacks; ++i) {
        const int d = (lane + LANES * i) * V;
        if (d < width) {
            if (weight) {
                float w[V];
#pragma unroll
                for (int e = 0; e < V; e += 4) ConvPack<float>::load(weight + d + e, w + e);
#pragma unroll
                for (int e = 0; e < V; ++e) v[i][e] = __fmul_rn(__fmul_rn(v[i][e], inv), w[e]);
            }
            ConvPack<T>::store(x + d, v[i]);
            if (dst) ConvPack<T>::store(dst + d, v[i]);
        }
    }
}

// grid (sequence slots of the step, channel blocks)
template <typename T>
__global__ void __launch_bounds__(128)
conv_tail_kernel(const T* __restrict__ raw, int ld, float* __restrict__ state, long long state_stride, long long tail_off,
                 const int32_t* __restrict__ q_start, const int32_t* __restrict__ q_len, const int32_t* __restrict__ state_slot, int C,
                 int taps) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x;
    const int len = q_len[seq];
    if (len <= 0) return;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int keep = taps - 1, start = q_start[seq];
    float* tail = state + static_cast<size_t>(state_slot[seq]) * state_stride + tail_off;
    float fresh[kConvMaxTaps - 1];
#pragma unroll
    for (int m = 0; m < kConvMaxTaps - 1; ++m) {
        if (m < keep) {
            const int src = len - keep + m;
            fresh[m] = src >= 0 ? to_f32(raw[static_cast<size_t>(start + src) * ld + c]) : tail[static_cast<size_t>(m + len) * C + c];
        }
    }
#pragma unroll
    for (int m = 0; m < kConvMaxTaps - 1; ++m)
        if (m < keep) tail[static_cast<size_t>(m) * C + c] = fresh[m];
}

}  // namespace stride

using namespace stride;

extern "C" {

int stride_conv_head_norm(const void* raw, int ld, void* out, int ld_out, const float* conv_w, int taps, const float* state,
                          long long state_stride, long long tail_off, const int32_t* seq_of_token, const int32_t* q_start,
                          const int32_t* state_slot, const float* wq, const float* wk, float eps, const int32_t* slot_mapping,
                          void* k_pages, void* v_pages, int tokens, int nq, int nkv, int hd, int vd, int page_size, int dtype,
                          cudaStream_t stream) {
    const long long C = static_cast<long long>(nq + nkv) * hd + static_cast<long long>(nkv) * vd;
    if (tokens < 0 || nq < 0 || nkv < 0 || hd <= 0 || vd <= 0 || page_size <= 0 || ld < C || ld_out < C || taps < 1) return STRIDE_BAD_ARGUMENT;
    if (taps > 1 && (!conv_w || !state || !q_start || !state_slot || state_stride < tail_off + (taps - 1) * C)) return STRIDE_BAD_ARGUMENT;
    if (slot_mapping != nullptr && (k_pages == nullptr || v_pages == nullptr)) return STRIDE_BAD_ARGUMENT;
    if (hd > kConvMaxHead || vd > kConvMaxHead || taps > kConvMaxTaps) return STRIDE_UNSUPPORTED;
    if (tokens == 0 || nq + nkv == 0) return 0;
    const dim3 grid(tokens, (nq + 2 * nkv + kConvWarps - 1) / kConvWarps);
    auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const int pack = dtype == STRIDE_DTYPE_F32 ? 4 : 8;
    const bool vec = hd % pack == 0 && vd % pack == 0 && ld % pack == 0 && ld_out % pack == 0 && aligned(raw) && aligned(out) &&
                     aligned(k_pages) && aligned(v_pages) && aligned(wq) && aligned(wk) && aligned(state) && aligned(conv_w) && state_stride % 4 == 0 &&
                     tail_off % 4 == 0;
    const bool halves = vec && hd <= 16 * pack && vd <= 16 * pack;       // two heads a warp
    const dim3 grid_h(tokens, ((nq + 2 * nkv + 1) / 2 + kConvWarps - 1) / kConvWarps);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(halves ? conv_head_norm_vec_kernel<float, 16> : vec ? conv_head_norm_vec_kernel<float, 32> : conv_head_norm_kernel<float>,
                       halves ? grid_h : grid, dim3(kConvWarps * 32), 0, stream, static_cast<const float*>(raw), ld,
                       static_cast<float*>(out), ld_out, conv_w, taps, state, state_stride, tail_off, seq_of_token, q_start, state_slot, wq, wk,
                       eps, slot_mapping, static_cast<float*>(k_pages), static_cast<float*>(v_pages), nq, nkv, hd, vd, page_size);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(halves ? conv_head_norm_vec_kernel<__nv_bfloat16, 16>
                       : vec  ? conv_head_norm_vec_kernel<__nv_bfloat16, 32>
                              : conv_head_norm_kernel<__nv_bfloat16>,
                       halves ? grid_h : grid, dim3(kConvWarps * 32), 0, stream, static_cast<const __nv_bfloat16*>(raw), ld,
                       static_cast<__nv_bfloat16*>(out), ld_out, conv_w, taps, state, state_stride, tail_off, seq_of_token, q_start, state_slot,
                       wq, wk, eps, slot_mapping, static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages), nq, nkv, hd, vd,
                       page_size);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_conv_tail(const void* raw, int ld, float* state, long long state_stride, long long tail_off, const int32_t* q_start,
                     const int32_t* q_len, const int32_t* state_slot, int num_seqs, int C, int taps, int dtype, cudaStream_t stream) {
    if (num_seqs < 0 || C <= 0 || ld < C || taps < 1 || !state || state_stride < tail_off + static_cast<long long>(taps - 1) * C)
        return STRIDE_BAD_ARGUMENT;
    if (taps > kConvMaxTaps || num_seqs > 0x7fffffff / 2) return STRIDE_UNSUPPORTED;
    if (num_seqs == 0 || taps == 1) return 0;
    const dim3 grid(num_seqs, (C + 127) / 128);
    if (grid.y > 65535) return STRIDE_UNSUPPORTED;
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(conv_tail_kernel<float>, grid, dim3(128), 0, stream, static_cast<const float*>(raw), ld, state, state_stride, tail_off,
                       q_start, q_len, state_slot, C, taps);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(conv_tail_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(raw), ld, state,
                       state_stride, tail_off, q_start, q_len, state_slot, C, taps);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
