// Norms whose statistic is the root mean square of a row, applied where the pre-norm decoder has none: on a sublayer's
// output before it joins the residual stream, and on the heads of queries, keys and values before they are used or kept.
// Statistics, scaling and the residual sum are float32; storage is float32 or bfloat16.
//
//   norm_add        residual[t] += m * w * y / sqrt(mean(y^2) + eps),  y = delta[t] (+ bias), and copy[t] = residual[t]
//                   in the compute dtype (what the next sublayer's products read). Without a delta it only makes the copy.
//                   With a second weight it also leaves next[t] = w' residual[t] / sqrt(mean(residual[t]^2) + eps'): the
//                   norm in front of the next sublayer, from the row while it is at hand.
//   qkv_unit_norm   for every token of a fused projection [q heads | k heads | v heads | anything else]: the bias is
//                   added, each query and key head (width hd) and each value head (width vd) is divided by its own root
//                   mean square (no weight; either norm can be switched off), written back in place, and keys and values
//                   go to the token's place in the pages ([page, kv_head, slot, width]) when a slot mapping is given.
//   rms_norm_cols   out[t] = x / sqrt(mean(x^2) + eps) * w for a column block x of a wider buffer (a latent between two
//                   products): one warp a row, float32 statistics.
// The order of every sum depends only on the row's width, never on the batch.
#include "common.cuh"

namespace stride {

template <typename T>
__global__ void norm_add_kernel(float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ bias,
                                const float* __restrict__ weight, T* __restrict__ copy, int hidden, float eps, float mult,
                                const float* __restrict__ next_weight, float next_eps, T* __restrict__ next_out) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float row_buf[];  // hidden floats, then 32 for the reduction
    float* scratch = row_buf + hidden;
    const size_t t = blockIdx.x;
    float* res = residual + t * hidden;
    if (delta == nullptr) {
        if (copy)
            for (int i = threadIdx.x; i < hidden; i += blockDim.x) copy[t * hidden + i] = from_f32<T>(res[i]);
        return;
    }
    const T* y = delta + t * hidden;
    float sq = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = to_f32(y[i]);
        if (bias) v = __fadd_rn(v, bias[i]);
        row_buf[i] = v;
        sq = fmaf(v, v, sq);
    }
    const float total = block_sum(sq, scratch);
    const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
    float sq2 = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float normed = __fmul_rn(__fmul_rn(row_buf[i], inv), weight[i]);
        const float x = __fadd_rn(res[i], __fmul_rn(mult, normed));
        res[i] = x;
        if (copy) copy[t * hidden + i] = from_f32<T>(x);
        if (next_out) {
            row_buf[i] = x;             // this thread's own entry: nobody else reads it before the next loop
            sq2 = fmaf(x, x, sq2);
        }
    }
    if (next_out == nullptr) return;
    const float inv2 = rsqrtf(block_sum(sq2, scratch) / static_cast<float>(hidden) + next_eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        next_out[t * hidden + i] = from_f32<T>(__fmul_rn(__fmul_rn(row_buf[i], inv2), next_weight[i]));
}

// Packs of 16 bytes of the compute dtype (8 bfloat16 or 4 float32) for the rows whose width is a whole number of them.
template <typename T>
struct Pack;
template <>
struct Pack<float> {
    static constexpr int V = 4;
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <>
struct Pack<__nv_bfloat16> {
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

// norm_add for rows of whole packs: the same sums in the same order per thread (a thread's elements are those of its
// packs), 16-byte accesses. A row's result depends on the width and the block size only.
template <typename T>
__global__ void norm_add_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ bias,
                                    const float* __restrict__ weight, T* __restrict__ copy, int hidden, float eps, float mult,
                                    const float* __restrict__ next_weight, float next_eps, T* __restrict__ next_out) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Pack<T>::V;
    extern __shared__ float row_buf[];  // hidden floats, then 32 for the reduction
    float* scratch = row_buf + hidden;
    const size_t t = blockIdx.x;
    float* res = residual + t * hidden;
    const int packs = hidden / V;
    if (delta == nullptr) {
        if (copy)
            for (int p = threadIdx.x; p < packs; p += blockDim.x) {
                float x[V];
#pragma unroll
                for (int j = 0; j < V; j += 4) Pack<float>::load(res + p * V + j, x + j);
                Pack<T>::store(copy + t * hidden + p * V, x);
            }
        return;
    }
    const T* y = delta + t * hidden;
    if (packs <= static_cast<int>(blockDim.x)) {
        // A pack a thread: everything the row needs is asked for before the sum, and nothing passes through shared
        // memory. The sums are those of the loops below (a thread's sum is its pack's).
        const int p = threadIdx.x;
        const bool on = p < packs;
        float v[V], w[V], x[V];
        float sq1 = 0.f;
        if (on) {
            Pack<T>::load(y + p * V, v);
#pragma unroll
            for (int j = 0; j < V; j += 4) {
                Pack<float>::load(weight + p * V + j, w + j);
                Pack<float>::load(res + p * V + j, x + j);
            }
            if (bias) {
                float b[V];
#pragma unroll
                for (int j = 0; j < V; j += 4) Pack<float>::load(bias + p * V + j, b + j);
#pragma unroll
                for (int j = 0; j < V; ++j) v[j] = __fadd_rn(v[j], b[j]);
            }
#pragma unroll
            for (int j = 0; j < V; ++j) sq1 = fmaf(v[j], v[j], sq1);
        }
        const float inv1 = rsqrtf(block_sum(sq1, scratch) / static_cast<float>(hidden) + eps);
        float sq2 = 0.f;
        if (on) {
#pragma unroll
            for (int j = 0; j < V; ++j) x[j] = __fadd_rn(x[j], __fmul_rn(mult, __fmul_rn(__fmul_rn(v[j], inv1), w[j])));
#pragma unroll
            for (int j = 0; j < V; j += 4) Pack<float>::store(res + p * V + j, x + j);
            if (copy) Pack<T>::store(copy + t * hidden + p * V, x);
#pragma unroll
            for (int j = 0; j < V; ++j) sq2 = fmaf(x[j], x[j], sq2);
        }
        if (next_out == nullptr) return;
        const float inv2 = rsqrtf(block_sum(sq2, scratch) / static_cast<float>(hidden) + next_eps);
        if (on) {
#pragma unroll
            for (int j = 0; j < V; j += 4) Pack<float>::load(next_weight + p * V + j, w + j);
#pragma unroll
            for (int j = 0; j < V; ++j) x[j] = __fmul_rn(__fmul_rn(x[j], inv2), w[j]);
            Pack<T>::store(next_out + t * hidden + p * V, x);
        }
        return;
    }
    float sq = 0.f;
    for (int p = threadIdx.x; p < packs; p += blockDim.x) {
        float v[V];
        Pack<T>::load(y + p * V, v);
        if (bias) {
            float b[V];
#pragma unroll
            for (int j = 0; j < V; j += 4) Pack<float>::load(bias + p * V + j, b + j);
#pragma unroll
            for (int j = 0; j < V; ++j) v[j] = __fadd_rn(v[j], b[j]);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) sq = fmaf(v[j], v[j], sq);
#pragma unroll
        for (int j = 0; j < V; j += 4) Pack<float>::store(row_buf + p * V + j, v + j);
    }
    const float total = block_sum(sq, scratch);
    const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
    float sq2 = 0.f;
    for (int p = threadIdx.x; p < packs; p += blockDim.x) {
        float v[V], w[V], x[V];
#pragma unroll
        for (int j = 0; j < V; j += 4) {
            Pack<float>::load(row_buf + p * V + j, v + j);
            Pack<float>::load(weight + p * V + j, w + j);
            Pack<float>::load(res + p * V + j, x + j);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) x[j] = __fadd_rn(x[j], __fmul_rn(mult, __fmul_rn(__fmul_rn(v[j], inv), w[j])));
#pragma unroll
        for (int j = 0; j < V; j += 4) Pack<float>::store(res + p * V + j, x + j);
        if (copy) Pack<T>::store(copy + t * hidden + p * V, x);
        if (next_out) {                 // this thread's own packs: nobody else reads them before the next loop
#pragma unroll
            for (int j = 0; j < V; j += 4) Pack<float>::store(row_buf + p * V + j, x + j);
#pragma unroll
            for (int j = 0; j < V; ++j) sq2 = fmaf(x[j], x[j], sq2);
        }
    }
    if (next_out == nullptr) return;
    const float inv2 = rsqrtf(block_sum(sq2, scratch) / static_cast<float>(hidden) + next_eps);
    for (int p = threadIdx.x; p < packs; p += blockDim.x) {
        float x[V], w[V];
#pragma unroll
        for (int j = 0; j < V; j += 4) {
            Pack<float>::load(row_buf + p * V + j, x + j);
            Pack<float>::load(next_weight + p * V + j, w + j);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) x[j] = __fmul_rn(__fmul_rn(x[j], inv2), w[j]);
        Pack<T>::store(next_out + t * hidden + p * V, x);
    }
}

constexpr int kNormWarps = 4;
constexpr int kMaxHead = 256;

template <typename T>
__global__ void __launch_bounds__(kNormWarps * 32)
qkv_unit_norm_kernel(T* __restrict__ qkv, int row_stride, const float* __restrict__ bias, const int32_t* __restrict__ slot_mapping,
                     T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv, int hd, int vd, int page_size, float eps,
                     int norm_qk, int norm_v) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * kNormWarps + warp;          // query heads, then key heads, then value heads
    if (head >= nq + 2 * nkv) return;
    const bool is_value = head >= nq + nkv;
    const int width = is_value ? vd : hd;
    const int column = is_value ? (nq + nkv) * hd + (head - nq - nkv) * vd : head * hd;
    T* x = qkv + static_cast<size_t>(t) * row_stride + column;
    float v[kMaxHead / 32];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxHead / 32; ++i) {
        const int d = lane + 32 * i;
        v[i] = 0.f;
        if (d < width) {
            v[i] = to_f32(x[d]);
            if (bias) v[i] = __fadd_rn(v[i], bias[column + d]);
            sq = fmaf(v[i], v[i], sq);
        }
    }
    const bool normed = is_value ? norm_v != 0 : norm_qk != 0;
    const float inv = normed ? rsqrtf(warp_sum(sq) / static_cast<float>(width) + eps) : 1.f;
    const int slot = (slot_mapping && head >= nq) ? slot_mapping[t] : -1;
    T* dst = nullptr;
    if (slot >= 0) {
        const int kvh = is_value ? head - nq - nkv : head - nq;
        dst = (is_value ? v_pages : k_pages) + ((static_cast<size_t>(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * width;
    }
#pragma unroll
    for (int i = 0; i < kMaxHead / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < width) {
            const T out = from_f32<T>(__fmul_rn(v[i], inv));
            x[d] = out;
            if (dst) dst[d] = out;
        }
    }
}

// qkv_unit_norm for heads of whole packs on 16-byte boundaries: a lane holds whole packs of its head (pack p of the head
// for p = lane, lane + 32, ...), so a warp moves a head in one or two 16-byte accesses a lane. The order of a head's sum
// depends on its width and on LANES only. LANES = 16: two heads a warp, for heads of at most 16 packs (the sum then stays
// inside a half warp).
template <typename T, int LANES>
__global__ void __launch_bounds__(kNormWarps * 32)
qkv_unit_norm_vec_kernel(T* __restrict__ qkv, int row_stride, const float* __restrict__ bias, const int32_t* __restrict__ slot_mapping,
                         T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv, int hd, int vd, int page_size, float eps,
                         int norm_qk, int norm_v) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Pack<T>::V;
    constexpr int kPacks = LANES == 32 ? kMaxHead / (32 * V) : 1;
    constexpr int kPerWarp = 32 / LANES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & (LANES - 1);
    const int t = blockIdx.x;
    // query heads, then key heads, then value heads
    const int head = (blockIdx.y * kNormWarps + warp) * kPerWarp + ((threadIdx.x & 31) / LANES);
    const bool live = head < nq + 2 * nkv;        // a half warp without a head still takes part in the shuffles
    const bool is_value = head >= nq + nkv;
    const int width = live ? (is_value ? vd : hd) : 0;
    const int column = is_value ? (nq + nkv) * hd + (head - nq - nkv) * vd : head * hd;
    T* x = qkv + static_cast<size_t>(t) * row_stride + (live ? column : 0);
    float v[kPacks][V];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < kPacks; ++i) {
        const int d = (lane + LANES * i) * V;
        if (d < width) {
            Pack<T>::load(x + d, v[i]);
            if (bias) {
                float b[V];
#pragma unroll
                for (int j = 0; j < V; j += 4) Pack<float>::load(bias + column + d + j, b + j);
#pragma unroll
                for (int j = 0; j < V; ++j) v[i][j] = __fadd_rn(v[i][j], b[j]);
            }
#pragma unroll
            for (int j = 0; j < V; ++j) sq = fmaf(v[i][j], v[i][j], sq);
        }
    }
    const bool normed = is_value ? norm_v != 0 : norm_qk != 0;
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float inv = normed && live ? rsqrtf(sq / static_cast<float>(width) + eps) : 1.f;
    const int slot = (slot_mapping && live && head >= nq) ? slot_mapping[t] : -1;
    T* dst = nullptr;
    if (slot >= 0) {
        const int kvh = is_value ? head - nq - nkv : head - nq;
        dst = (is_value ? v_pages : k_pages) + ((static_cast<size_t>(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * width;
    }
#pragma unroll
    for (int i = 0; i < kPacks; ++i) {
        const int d = (lane + LANES * i) * V;
        if (d < width) {
#pragma unroll
            for (int j = 0; j < V; ++j) v[i][j] = __fmul_rn(v[i][j], inv);
            Pack<T>::store(x + d, v[i]);
            if (dst) Pack<T>::store(dst + d, v[i]);
        }
    }
}

// x: [rows, ld] from column 0 on (the caller offsets the pointer); out: [rows, ld_out]. One warp a row.
template <typename T>
__global__ void __launch_bounds__(128)
rms_norm_cols_kernel(const T* __restrict__ x, int ld, const float* __restrict__ weight, T* __restrict__ out, int ld_out, int rows, int width,
                     float eps) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= rows) return;
    const T* src = x + static_cast<size_t>(r) * ld;
    float sq = 0.f;
    for (int i = lane; i < width; i += 32) {
        const float v = to_f32(src[i]);
        sq = fmaf(v, v, sq);
    }
    const float inv = rsqrtf(warp_sum(sq) / static_cast<float>(width) + eps);
    T* dst = out + static_cast<size_t>(r) * ld_out;
    for (int i = lane; i < width; i += 32) dst[i] = from_f32<T>(__fmul_rn(__fmul_rn(to_f32(src[i]), inv), weight[i]));
}

}  // namespace stride

using namespace stride;

extern "C" {

int stride_norm_add(float* residual, const void* delta, const float* bias, const float* weight, void* copy, int tokens, int hidden,
                    float eps, float mult, const float* next_weight, float next_eps, void* next_out, int dtype, cudaStream_t stream) {
    if (tokens < 0 || hidden <= 0 || (delta != nullptr && weight == nullptr)) return STRIDE_BAD_ARGUMENT;
    if (next_out != nullptr && (next_weight == nullptr || delta == nullptr)) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const int threads = hidden >= 4096 ? 512 : hidden >= 1024 ? 256 : 128;
    const size_t smem = (static_cast<size_t>(hidden) + 32) * sizeof(float);
    if (smem > 200 * 1024) return STRIDE_UNSUPPORTED;
    auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool vec = hidden % 8 == 0 && aligned(residual) && aligned(delta) && aligned(bias) && aligned(weight) && aligned(copy) &&
                     aligned(next_weight) && aligned(next_out);
    if (dtype == STRIDE_DTYPE_F32) {
        auto kernel = vec ? norm_add_vec_kernel<float> : norm_add_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        stride::launch(kernel, dim3(tokens), dim3(threads), smem, stream, residual, static_cast<const float*>(delta), bias,
                       weight, static_cast<float*>(copy), hidden, eps, mult, next_weight, next_eps, static_cast<float*>(next_out));
    } else if (dtype == STRIDE_DTYPE_BF16) {
        auto kernel = vec ? norm_add_vec_kernel<__nv_bfloat16> : norm_add_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        stride::launch(kernel, dim3(tokens), dim3(threads), smem, stream, residual,
                       static_cast<const __nv_bfloat16*>(delta), bias, weight, static_cast<__nv_bfloat16*>(copy), hidden, eps, mult,
                       next_weight, next_eps, static_cast<__nv_bfloat16*>(next_out));
    } else {
        return STRIDE_BAD_ARGUMENT;
    }
    return STRIDE_LAUNCH_STATUS();
}

int stride_rms_norm_cols(const void* x, int ld, const float* weight, void* out, int ld_out, int rows, int width, float eps, int dtype,
                         cudaStream_t stream) {
    if (rows < 0 || width <= 0 || ld < width || ld_out < width || !weight) return STRIDE_BAD_ARGUMENT;
    if (rows == 0) return 0;
    const dim3 grid((rows + 3) / 4);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(rms_norm_cols_kernel<float>, grid, dim3(128), 0, stream, static_cast<const float*>(x), ld, weight, static_cast<float*>(out),
                       ld_out, rows, width, eps);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(rms_norm_cols_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(x), ld, weight,
                       static_cast<__nv_bfloat16*>(out), ld_out, rows, width, eps);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_qkv_unit_norm(void* qkv, int row_stride, const float* bias, const int32_t* slot_mapping, void* k_pages, void* v_pages,
                         int tokens, int nq, int nkv, int hd, int vd, int page_size, float eps, int norm_qk, int norm_v, int dtype,
                         cudaStream_t stream) {
    if (tokens < 0 || nq < 0 || nkv < 0 || hd <= 0 || vd <= 0 || page_size <= 0 || row_stride < (nq + nkv) * hd + nkv * vd)
        return STRIDE_BAD_ARGUMENT;
    if (slot_mapping != nullptr && (k_pages == nullptr || v_pages == nullptr)) return STRIDE_BAD_ARGUMENT;
    if (hd > kMaxHead || vd > kMaxHead) return STRIDE_UNSUPPORTED;
    if (tokens == 0 || nq + nkv == 0) return 0;
    const dim3 grid(tokens, (nq + 2 * nkv + kNormWarps - 1) / kNormWarps);
    auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const int pack = dtype == STRIDE_DTYPE_F32 ? 4 : 8;
    const bool vec = hd % pack == 0 && vd % pack == 0 && row_stride % pack == 0 && aligned(qkv) && aligned(bias) && aligned(k_pages) &&
                     aligned(v_pages);
    const bool halves = vec && hd <= 16 * pack && vd <= 16 * pack;       // two heads a warp
    const dim3 grid_h(tokens, ((nq + 2 * nkv + 1) / 2 + kNormWarps - 1) / kNormWarps);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(halves ? qkv_unit_norm_vec_kernel<float, 16> : vec ? qkv_unit_norm_vec_kernel<float, 32> : qkv_unit_norm_kernel<float>,
                       halves ? grid_h : grid, dim3(kNormWarps * 32), 0, stream, static_cast<float*>(qkv), row_stride, bias, slot_mapping,
                       static_cast<float*>(k_pages), static_cast<float*>(v_pages), nq, nkv, hd, vd, page_size, eps, norm_qk, norm_v);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(halves ? qkv_unit_norm_vec_kernel<__nv_bfloat16, 16>
                       : vec  ? qkv_unit_norm_vec_kernel<__nv_bfloat16, 32>
                              : qkv_unit_norm_kernel<__nv_bfloat16>,
                       halves ? grid_h : grid, dim3(kNormWarps * 32), 0, stream, static_cast<__nv_bfloat16*>(qkv), row_stride, bias,
                       slot_mapping, static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages), nq, nkv, hd, vd, page_size,
                       eps, norm_qk, norm_v);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
