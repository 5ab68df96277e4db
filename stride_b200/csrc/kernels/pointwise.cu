// Small elementwise kernels that several mixers, feed-forwards and heads share. All arithmetic is float32; storage is
// float32 or bfloat16. One 16-byte pack per thread where pointers and sizes allow it (the form that streams fastest
// here), one element per thread otherwise.
//
//   gated_act     out = act(gate) * up for [tokens, 2 * inter] whose gate and up columns alternate in blocks
//                 (the layout of the fused gate/up product); act: 0 SiLU, 1 the tanh form of GELU, 2 the clamped
//                 form g' sigmoid(a g') (u' + 1) with g' = min(g, limit) and u' = clamp(u, -limit, limit)
//   sigmoid_gate  x *= sigmoid(g)
//   head_gate     x[t, h, :] *= sigmoid(g[t, h]): one gate per head, read from a column block of a wider buffer
//   add_sinusoid  x[t, 2i] += sin(p_t f_i), x[t, 2i + 1] += cos(p_t f_i) with float64 angles, and optionally the
//                 sum's copy in the compute dtype
//   softcap       x = c tanh(x / c)            (float32, in place: logits)
//   tanh_inplace  x = tanh(x)
//   weighted_sum  out = sa * a + sb * b        (the sum of two branches; out may be a or b)
//   stream_concat out[t] = [x[t] rounded to the compute dtype | y[t]]: the float32 stream beside a second input, as the
//                 operand of one product over both
//   add_row_vector x[t, :] += b for every live row (float32)
#include "common.cuh"

namespace stride {

template <typename T>
struct Vec;
template <>
struct Vec<float> {
    static constexpr int V = 4;
    float v[4];
    __device__ __forceinline__ void load(const float* p) {
        const float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <>
struct Vec<__nv_bfloat16> {
    static constexpr int V = 8;
    float v[8];
    __device__ __forceinline__ void load(const __nv_bfloat16* p) {
        const uint4 r = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
    __device__ __forceinline__ void store(__nv_bfloat16* p) const {
        uint4 r;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = r;
    }
};

__device__ __forceinline__ float act_f(float g, int act) {
    if (act == 1) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.f + expf(-g));
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
// act(gate) * up for every activation; `limit` and `alpha` only matter to the clamped form.
__device__ __forceinline__ float gated_f(float g, float u, int act, float limit, float alpha) {
    if (act == 2) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g * sigmoid_f(alpha * g) * (u + 1.f);
    }
    return act_f(g, act) * u;
}

template <typename T>
__global__ void gated_act_vec_kernel(const T* __restrict__ in, T* __restrict__ out, int inter, int block, int act, float limit, float alpha, size_t packs) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Vec<T>::V;
    const int per_row = inter / V;
    const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (idx >= packs) return;
    const size_t t = idx / per_row;
    const int i = static_cast<int>(idx - t * per_row) * V;
    const size_t at = t * 2 * inter + static_cast<size_t>(i / block) * 2 * block + i % block;
    Vec<T> g, u;
    g.load(in + at);
    u.load(in + at + block);
#pragma unroll
    for (int j = 0; j < V; ++j) g.v[j] = gated_f(g.v[j], u.v[j], act, limit, alpha);
    g.store(out + t * inter + i);
}

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ in, T* __restrict__ out, int inter, int block, int act, float limit, float alpha, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / inter;
    const int i = static_cast<int>(idx - t * inter);
    const size_t at = t * 2 * inter + static_cast<size_t>(i / block) * 2 * block + i % block;
    out[idx] = from_f32<T>(gated_f(to_f32(in[at]), to_f32(in[at + block]), act, limit, alpha));
}

// op: 0  x *= sigmoid(g);  1  x = cap * tanh(x / cap);  2  x = tanh(x)
template <typename T>
__global__ void unary_vec_kernel(T* __restrict__ x, const T* __restrict__ g, int op, float cap, size_t packs) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Vec<T>::V;
    const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (idx >= packs) return;
    Vec<T> a, b;
    a.load(x + idx * V);
    if (op == 0) b.load(g + idx * V);
#pragma unroll
    for (int j = 0; j < V; ++j)
        a.v[j] = op == 0 ? a.v[j] * sigmoid_f(b.v[j]) : op == 1 ? cap * tanhf(a.v[j] / cap) : tanhf(a.v[j]);
    a.store(x + idx * V);
}

template <typename T>
__global__ void unary_kernel(T* __restrict__ x, const T* __restrict__ g, int op, float cap, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (idx >= total) return;
    const float a = to_f32(x[idx]);
    x[idx] = from_f32<T>(op == 0 ? a * sigmoid_f(to_f32(g[idx])) : op == 1 ? cap * tanhf(a / cap) : tanhf(a));
}

template <typename T>
__global__ void weighted_sum_vec_kernel(T* out, const T* a, float sa, const T* b, float sb, size_t packs) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Vec<T>::V;
    const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (idx >= packs) return;
    Vec<T> x, y;
    x.load(a + idx * V);
    y.load(b + idx * V);
#pragma unroll
    for (int j = 0; j < V; ++j) x.v[j] = fmaf(sb, y.v[j], sa * x.v[j]);
    x.store(out + idx * V);
}

template <typename T>
__global__ void weighted_sum_kernel(T* out, const T* a, float sa, const T* b, float sb, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (idx >= total) return;
    out[idx] = from_f32<T>(fmaf(sb, to_f32(b[idx]), sa * to_f32(a[idx])));
}

// x: [tokens, heads, width]; the gate of head h of token t is g[t * g_stride + h].
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, const T* __restrict__ g, int g_stride, int heads, int width, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (idx >= total) return;
    const size_t th = idx / width;
    const size_t t = th / heads;
    const int h = static_cast<int>(th - t * heads);
    x[idx] = from_f32<T>(to_f32(x[idx]) * sigmoid_f(to_f32(g[t * g_stride + h])));
}

// The same, 16 bytes a thread, for head widths that are whole packs (a pack then lies inside one head).
template <typename T>
__global__ void head_gate_vec_kernel(T* __restrict__ x, const T* __restrict__ g, int g_stride, int heads, int packs_per_head, size_t packs) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Vec<T>::V;
    for (size_t p = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; p < packs; p += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t th = p / packs_per_head;
        const size_t t = th / heads;
        const int h = static_cast<int>(th - t * heads);
        const float s = sigmoid_f(to_f32(g[t * g_stride + h]));
        Vec<T> v;
        v.load(x + p * V);
#pragma unroll
        for (int j = 0; j < V; ++j) v.v[j] *= s;
        v.store(x + p * V);
    }
}

// freq: float64 [ceil(width / 2)]. Rows of padded tokens (seq_of_token < 0) are left alone.
template <typename T>
__global__ void add_sinusoid_kernel(float* __restrict__ x, T* __restrict__ copy, const int32_t* __restrict__ positions,
                                    const int32_t* __restrict__ seq_of_token, const double* __restrict__ freq, int width) {
    pdl_trigger();
    pdl_wait();
    const size_t t = blockIdx.x;
    const bool live = seq_of_token == nullptr || seq_of_token[t] >= 0;
    const double p = static_cast<double>(positions[t]);
    // a pair a thread, the pairs of a row spread over blockIdx.y: the float64 sine and cosine are the kernel's time
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; 2 * i < width; i += gridDim.y * blockDim.x) {
        double s = 0.0, c = 0.0;
        if (live) sincos(p * freq[i], &s, &c);
        const size_t at = t * width + 2 * i;
        const float a = __fadd_rn(x[at], static_cast<float>(s));
        x[at] = a;
        if (copy) copy[at] = from_f32<T>(a);
        if (2 * i + 1 < width) {
            const float b = __fadd_rn(x[at + 1], static_cast<float>(c));
            x[at + 1] = b;
            if (copy) copy[at + 1] = from_f32<T>(b);
        }
    }
}

template <typename T>
int weighted(void* out, const void* a, float sa, const void* b, float sb, long long n, cudaStream_t stream) {
    constexpr int V = Vec<T>::V;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b);
    if (bits % 16 == 0 && n % V == 0) {
        const size_t packs = static_cast<size_t>(n) / V;
        stride::launch(weighted_sum_vec_kernel<T>, dim3(static_cast<unsigned>((packs + 127) / 128)), dim3(128), 0, stream, static_cast<T*>(out),
                       static_cast<const T*>(a), sa, static_cast<const T*>(b), sb, packs);
    } else {
        stride::launch(weighted_sum_kernel<T>, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, stream, static_cast<T*>(out),
                       static_cast<const T*>(a), sa, static_cast<const T*>(b), sb, static_cast<size_t>(n));
    }
    return STRIDE_LAUNCH_STATUS();
}

template <typename T>
int unary(void* x, const void* g, int op, float cap, long long n, cudaStream_t stream) {
    constexpr int V = Vec<T>::V;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g);
    if (bits % 16 == 0 && n % V == 0) {
        const size_t packs = static_cast<size_t>(n) / V;
        stride::launch(unary_vec_kernel<T>, dim3(static_cast<unsigned>((packs + 127) / 128)), dim3(128), 0, stream, static_cast<T*>(x),
                       static_cast<const T*>(g), op, cap, packs);
    } else {
        stride::launch(unary_kernel<T>, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, stream, static_cast<T*>(x),
                       static_cast<const T*>(g), op, cap, static_cast<size_t>(n));
    }
    return STRIDE_LAUNCH_STATUS();
}

template <typename T>
int gated(const void* in, void* out, int tokens, int inter, int block, int act, float limit, float alpha, cudaStream_t stream) {
    constexpr int V = Vec<T>::V;
    const size_t total = static_cast<size_t>(tokens) * inter;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out);
    if (bits % 16 == 0 && block % V == 0) {
        const size_t packs = total / V;
        stride::launch(gated_act_vec_kernel<T>, dim3(static_cast<unsigned>((packs + 127) / 128)), dim3(128), 0, stream,
                       static_cast<const T*>(in), static_cast<T*>(out), inter, block, act, limit, alpha, packs);
    } else {
        stride::launch(gated_act_kernel<T>, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, stream, static_cast<const T*>(in),
                       static_cast<T*>(out), inter, block, act, limit, alpha, total);
    }
    return STRIDE_LAUNCH_STATUS();
}

template <typename T>
__global__ void stream_concat_kernel(const float* __restrict__ x, const T* __restrict__ y, T* __restrict__ out, int width, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / (2 * static_cast<size_t>(width));
    const int c = static_cast<int>(i - t * 2 * width);
    out[i] = c < width ? from_f32<T>(x[t * width + c]) : y[t * width + (c - width)];
}

__global__ void add_row_vector_kernel(float* __restrict__ x, const float* __restrict__ b, const int32_t* __restrict__ seq_of_token, int width,
                                      size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / width;
    if (seq_of_token && seq_of_token[t] < 0) return;
    x[i] = __fadd_rn(x[i], b[i - t * width]);
}

}  // namespace stride

using namespace stride;

extern "C" {

int stride_gated_act(const void* in, void* out, int tokens, int inter, int block, int act, float limit, float alpha, int dtype,
                     cudaStream_t stream) {
    if (tokens < 0 || inter <= 0 || block <= 0 || inter % block || act < 0 || act > 2) return STRIDE_BAD_ARGUMENT;
    if (static_cast<size_t>(tokens) * inter / 4 / 128 > 0x7fffffffull) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    if (dtype == STRIDE_DTYPE_F32) return gated<float>(in, out, tokens, inter, block, act, limit, alpha, stream);
    if (dtype == STRIDE_DTYPE_BF16) return gated<__nv_bfloat16>(in, out, tokens, inter, block, act, limit, alpha, stream);
    return STRIDE_BAD_ARGUMENT;
}

int stride_head_gate(void* x, const void* g, int g_stride, int tokens, int heads, int width, int dtype, cudaStream_t stream) {
    if (tokens < 0 || heads <= 0 || width <= 0 || g_stride < heads) return STRIDE_BAD_ARGUMENT;
    const size_t total = static_cast<size_t>(tokens) * heads * width;
    if (total / 256 > 0x7fffffffull) return STRIDE_UNSUPPORTED;
    if (total == 0) return 0;
    const int pack = dtype == STRIDE_DTYPE_F32 ? 4 : 8;
    if ((dtype == STRIDE_DTYPE_F32 || dtype == STRIDE_DTYPE_BF16) && width % pack == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0) {
        const size_t packs = total / pack;
        const dim3 vgrid(static_cast<unsigned>(packs / 256 >= 148 * 16 ? 148 * 16 : (packs + 255) / 256));
        if (dtype == STRIDE_DTYPE_F32)
            stride::launch(head_gate_vec_kernel<float>, vgrid, dim3(256), 0, stream, static_cast<float*>(x), static_cast<const float*>(g),
                           g_stride, heads, width / pack, packs);
        else
            stride::launch(head_gate_vec_kernel<__nv_bfloat16>, vgrid, dim3(256), 0, stream, static_cast<__nv_bfloat16*>(x),
                           static_cast<const __nv_bfloat16*>(g), g_stride, heads, width / pack, packs);
        return STRIDE_LAUNCH_STATUS();
    }
    const dim3 grid(static_cast<unsigned>((total + 255) / 256));
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(head_gate_kernel<float>, grid, dim3(256), 0, stream, static_cast<float*>(x), static_cast<const float*>(g), g_stride,
                       heads, width, total);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(head_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, static_cast<__nv_bfloat16*>(x),
                       static_cast<const __nv_bfloat16*>(g), g_stride, heads, width, total);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_add_sinusoid(float* x, void* copy, const int32_t* positions, const int32_t* seq_of_token, const double* freq, int tokens,
                        int width, int dtype, cudaStream_t stream) {
    if (tokens < 0 || width <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const int slices = ((width + 1) / 2 + 127) / 128;
    const dim3 grid(tokens, slices < 65535 ? slices : 65535);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(add_sinusoid_kernel<float>, grid, dim3(128), 0, stream, x, static_cast<float*>(copy), positions, seq_of_token,
                       freq, width);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(add_sinusoid_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, x, static_cast<__nv_bfloat16*>(copy), positions,
                       seq_of_token, freq, width);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_pointwise(void* x, const void* g, int op, float cap, long long n, int dtype, cudaStream_t stream) {
    if (n < 0 || op < 0 || op > 2 || (op == 0 && g == nullptr) || (op == 1 && !(cap > 0.f))) return STRIDE_BAD_ARGUMENT;
    if (n / 4 / 128 > 0x7fffffffll) return STRIDE_UNSUPPORTED;
    if (n == 0) return 0;
    if (dtype == STRIDE_DTYPE_F32) return unary<float>(x, g, op, cap, n, stream);
    if (dtype == STRIDE_DTYPE_BF16) return unary<__nv_bfloat16>(x, g, op, cap, n, stream);
    return STRIDE_BAD_ARGUMENT;
}

int stride_stream_concat(const float* x, const void* y, void* out, int tokens, int width, int dtype, cudaStream_t stream) {
    if (tokens < 0 || width <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const size_t total = static_cast<size_t>(tokens) * 2 * width;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(stream_concat_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, static_cast<const float*>(y), static_cast<float*>(out),
                       width, total);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(stream_concat_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, x, static_cast<const __nv_bfloat16*>(y),
                       static_cast<__nv_bfloat16*>(out), width, total);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_add_row_vector(float* x, const float* b, const int32_t* seq_of_token, int tokens, int width, cudaStream_t stream) {
    if (tokens < 0 || width <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const size_t total = static_cast<size_t>(tokens) * width;
    stride::launch(add_row_vector_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, stream, x, b, seq_of_token, width, total);
    return STRIDE_LAUNCH_STATUS();
}

int stride_weighted_sum(void* out, const void* a, float sa, const void* b, float sb, long long n, int dtype, cudaStream_t stream) {
    if (n < 0) return STRIDE_BAD_ARGUMENT;
    if (n / 4 / 128 > 0x7fffffffll) return STRIDE_UNSUPPORTED;
    if (n == 0) return 0;
    if (dtype == STRIDE_DTYPE_F32) return weighted<float>(out, a, sa, b, sb, n, stream);
    if (dtype == STRIDE_DTYPE_BF16) return weighted<__nv_bfloat16>(out, a, sa, b, sb, n, stream);
    return STRIDE_BAD_ARGUMENT;
}

}  // extern "C"
