// A residual stream kept in float whatever the activations' element type is, and what works on it:
//
//   embed_positions : h[t, :] = float(table[token_t, :]) * scale + float(pos_table[position_t, :])
//                     (a scaled token embedding plus a learned position vector; optionally a second copy of h)
//   resid_update    : h[t, :] <- ((h + (d1 + d2)) + e[t, :]) + vec      every addend optional, sums in float, in place;
//                     with a norm weight w also  out[t, :] = T( h * (1 / sqrt(mean(h^2) + eps)) * w ): RMSNorm with one
//                     rounding, at the store.  One kernel serves the plain norm, the residual add fused with the next
//                     norm, and the input of a repeated pass (the embedding output and a per-pass vector added).
//   gelu_tanh       : out = T( 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))) ), z = float(x)
//   write_rows      : rows of a packed projection into cache pages [page, heads, slot in page, width] (a cache that
//                     holds one vector per token and head: keys that also serve as values)
//   norm_add        : h[t, :] <- [h[t, :] +] (y + b) / sqrt(mean((y + b)^2) + eps) * w, with y a sublayer's output and b an
//                     optional bias: the norm sits behind the sublayer and only its result joins the stream.  A copy of the
//                     new stream in the activations' type is written beside it (what the next sublayer's products read).
//   bias_act        : out = T( act(x + b) ), act = identity | relu(z)^2 | tanh-GELU
//   gated_norm      : out[t, g, j] = T( o / sqrt(mean_j(o[t, g, :]^2) + eps) * w[j] * sigmoid(gate[t, g, j]) ) over groups of
//                     (or times silu(gate): `gate_act` = 1) over groups of
//                     equal size (one group: a norm over the whole row; one group per head: a norm per head with a weight
//                     that the heads share); o is float, the gate a column range of a packed projection
//
// T is the activations' element type (float or bf16); deltas d1, d2 and the norm's output have it.
#include "common.cuh"

namespace cvb {

template <typename T>
__global__ void embed_positions_kernel(float* __restrict__ out, float* __restrict__ out2, const T* __restrict__ table,
                                       const T* __restrict__ pos_table, const int* __restrict__ tokens,
                                       const int* __restrict__ positions, int D, int V, int P, float scale,
                                       int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int64_t t = blockIdx.x;
    int tok = tokens[t], pos = positions[t];
    if (tok < 0 || tok >= V) {
        if (threadIdx.x == 0) atomicExch(err, 1);
        tok = tok < 0 ? 0 : V - 1;
    }
    if (pos_table != nullptr && (pos < 0 || pos >= P)) {
        if (threadIdx.x == 0) atomicExch(err, 3);
        pos = pos < 0 ? 0 : P - 1;
    }
    const T* row = table + static_cast<int64_t>(tok) * D;
    const T* prow = pos_table ? pos_table + static_cast<int64_t>(pos) * D : nullptr;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = to_float(row[i]) * scale;
        if (prow) v += to_float(prow[i]);
        out[t * D + i] = v;
        if (out2) out2[t * D + i] = v;
    }
}

constexpr int kUpdateThreads = 128;

template <typename T>
__global__ void __launch_bounds__(kUpdateThreads)
resid_update_kernel(float* h, const T* __restrict__ d1, const T* __restrict__ d2, const float* __restrict__ e,
                    const float* __restrict__ vec, const float* __restrict__ w, T* __restrict__ out, int D, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    float* hr = h + row * D;
    const bool changes = d1 != nullptr || e != nullptr || vec != nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += kUpdateThreads) {
        float v = hr[i];
        if (d1) {
            float a = to_float(d1[row * D + i]);
            if (d2) a += to_float(d2[row * D + i]);
            v += a;
        }
        if (e) v += e[row * D + i];
        if (vec) v += vec[i];
        if (changes) hr[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (w == nullptr) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / static_cast<float>(D) + eps);
    // a thread reads back only what it wrote itself
    for (int i = threadIdx.x; i < D; i += kUpdateThreads) out[row * D + i] = from_float<T>(hr[i] * inv * w[i]);
}

// Rows whose length is a multiple of four floats: the row stays in registers between the sum and the norm.
constexpr int kUpdateChunks = 8;       // rows up to 128 * 8 * 4 = 4,096 floats

template <typename T>
__global__ void __launch_bounds__(kUpdateThreads)
resid_update_vec_kernel(float* h, const T* __restrict__ d1, const T* __restrict__ d2, const float* __restrict__ e,
                        const float* __restrict__ vec, const float* __restrict__ w, T* __restrict__ out, int D, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const int n_chunks = D / 4;
    const bool changes = d1 != nullptr || e != nullptr || vec != nullptr;
    float4 val[kUpdateChunks];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kUpdateChunks; ++k) {
        const int c = threadIdx.x + k * kUpdateThreads;
        if (c < n_chunks) {
            float4 v = *reinterpret_cast<const float4*>(h + row * D + c * 4);
            if (d1) {
                const T* p1 = d1 + row * D + c * 4;
                float a0 = to_float(p1[0]), a1 = to_float(p1[1]), a2 = to_float(p1[2]), a3 = to_float(p1[3]);
                if (d2) {
                    const T* p2 = d2 + row * D + c * 4;
                    a0 += to_float(p2[0]); a1 += to_float(p2[1]); a2 += to_float(p2[2]); a3 += to_float(p2[3]);
                }
                v.x += a0; v.y += a1; v.z += a2; v.w += a3;
            }
            if (e) {
                const float4 a = *reinterpret_cast<const float4*>(e + row * D + c * 4);
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
            if (vec) {
                const float4 a = *reinterpret_cast<const float4*>(vec + c * 4);
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
            if (changes) *reinterpret_cast<float4*>(h + row * D + c * 4) = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            val[k] = v;
        }
    }
    if (w == nullptr) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
    for (int k = 0; k < kUpdateChunks; ++k) {
        const int c = threadIdx.x + k * kUpdateThreads;
        if (c < n_chunks) {
            const float4 ww = *reinterpret_cast<const float4*>(w + c * 4);
            T* o = out + row * D + c * 4;
            o[0] = from_float<T>(val[k].x * inv * ww.x);
            o[1] = from_float<T>(val[k].y * inv * ww.y);
            o[2] = from_float<T>(val[k].z * inv * ww.z);
            o[3] = from_float<T>(val[k].w * inv * ww.w);
        }
    }
}

__device__ __forceinline__ float gelu_tanh_of(float z) {
    const float inner = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.f + tanhf(inner));
}

template <typename T>
__global__ void gelu_tanh_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t n) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        out[i] = from_float<T>(gelu_tanh_of(to_float(x[i])));
}

// bf16, eight elements per thread and step
__global__ void gelu_tanh_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, int64_t n_chunks) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_chunks;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + i * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        uint4 res;
        __nv_bfloat162* r = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __bfloat1622float2(h[k]);
            r[k] = __floats2bfloat162_rn(gelu_tanh_of(f.x), gelu_tanh_of(f.y));
        }
        *reinterpret_cast<uint4*>(out + i * 8) = res;
    }
}

// The norm behind a sublayer: only the normed output joins the stream.
template <typename T>
__global__ void __launch_bounds__(kUpdateThreads)
norm_add_kernel(float* __restrict__ h, const T* __restrict__ y, const float* __restrict__ bias, const float* __restrict__ w,
                T* __restrict__ copy, int D, float eps, int accumulate) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const T* yr = y + row * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += kUpdateThreads) {
        const float v = to_float(yr[i]) + (bias ? bias[i] : 0.f);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / static_cast<float>(D) + eps);
    for (int i = threadIdx.x; i < D; i += kUpdateThreads) {
        const float v = to_float(yr[i]) + (bias ? bias[i] : 0.f);
        const float r = (accumulate ? h[row * D + i] : 0.f) + v * inv * w[i];
        h[row * D + i] = r;
        if (copy) copy[row * D + i] = from_float<T>(r);
    }
}

// Rows whose length is a multiple of four: every load is asked for before the first is used, the row stays in registers.
template <typename T>
__global__ void __launch_bounds__(kUpdateThreads)
norm_add_vec_kernel(float* __restrict__ h, const T* __restrict__ y, const float* __restrict__ bias, const float* __restrict__ w,
                    T* __restrict__ copy, int D, float eps, int accumulate) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const int n_chunks = D / 4;
    float4 val[kUpdateChunks], old[kUpdateChunks], ww[kUpdateChunks];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kUpdateChunks; ++k) {
        const int c = threadIdx.x + k * kUpdateThreads;
        if (c < n_chunks) {
            const T* py = y + row * D + c * 4;
            float4 v = make_float4(to_float(py[0]), to_float(py[1]), to_float(py[2]), to_float(py[3]));
            if (bias) {
                const float4 b = *reinterpret_cast<const float4*>(bias + c * 4);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            val[k] = v;
            ww[k] = *reinterpret_cast<const float4*>(w + c * 4);
            old[k] = accumulate ? *reinterpret_cast<const float4*>(h + row * D + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
    for (int k = 0; k < kUpdateChunks; ++k) {
        const int c = threadIdx.x + k * kUpdateThreads;
        if (c < n_chunks) {
            float4 r;
            r.x = old[k].x + val[k].x * inv * ww[k].x;
            r.y = old[k].y + val[k].y * inv * ww[k].y;
            r.z = old[k].z + val[k].z * inv * ww[k].z;
            r.w = old[k].w + val[k].w * inv * ww[k].w;
            *reinterpret_cast<float4*>(h + row * D + c * 4) = r;
            if (copy) {
                T* o = copy + row * D + c * 4;
                o[0] = from_float<T>(r.x); o[1] = from_float<T>(r.y); o[2] = from_float<T>(r.z); o[3] = from_float<T>(r.w);
            }
        }
    }
}

template <typename T>
__global__ void bias_act_kernel(T* __restrict__ out, const T* __restrict__ x, const float* __restrict__ bias, int64_t n, int D,
                                int act) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        float z = to_float(x[i]) + (bias ? bias[i % D] : 0.f);
        if (act == 1) { z = fmaxf(z, 0.f); z = z * z; }
        else if (act == 2) z = gelu_tanh_of(z);
        out[i] = from_float<T>(z);
    }
}

// bf16 rows whose length is a multiple of eight: eight elements per thread and step
__global__ void bias_act_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, const float* __restrict__ bias,
                                       int64_t n_chunks, int D, int act) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_chunks;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + i * 8);
        const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const int c0 = static_cast<int>((i * 8) % D);
        uint4 res;
        __nv_bfloat162* r = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 f = __bfloat1622float2(hx[k]);
            if (bias) { f.x += bias[c0 + 2 * k]; f.y += bias[c0 + 2 * k + 1]; }
            if (act == 1) { f.x = fmaxf(f.x, 0.f); f.x *= f.x; f.y = fmaxf(f.y, 0.f); f.y *= f.y; }
            else if (act == 2) { f.x = gelu_tanh_of(f.x); f.y = gelu_tanh_of(f.y); }
            r[k] = __floats2bfloat162_rn(f.x, f.y);
        }
        *reinterpret_cast<uint4*>(out + i * 8) = res;
    }
}

// Large groups: a block per (token, group).
template <typename T>
__global__ void __launch_bounds__(kUpdateThreads)
gated_norm_block_kernel(T* __restrict__ out, const float* __restrict__ o, const T* __restrict__ gate, int gate_stride,
                        const float* __restrict__ w, int groups, int G, float eps, int gate_act) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int64_t row = blockIdx.x;
    const int g = blockIdx.y;
    const float* og = o + (row * groups + g) * G;
    float ss = 0.f;
    for (int j = threadIdx.x; j < G; j += kUpdateThreads) ss = fmaf(og[j], og[j], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / static_cast<float>(G) + eps);
    for (int j = threadIdx.x; j < G; j += kUpdateThreads) {
        const float z = to_float(gate[row * gate_stride + g * G + j]);
        out[(row * groups + g) * G + j] = from_float<T>(og[j] * inv * w[j] * (gate_act ? z : 1.f) * (1.f / (1.f + expf(-z))));
    }
}

// Small groups: a block per token and four groups; a warp takes a group.
template <typename T>
__global__ void __launch_bounds__(kUpdateThreads)
gated_norm_kernel(T* __restrict__ out, const float* __restrict__ o, const T* __restrict__ gate, int gate_stride,
                  const float* __restrict__ w, int groups, int G, float eps, int gate_act) {
    pdl_trigger();
    pdl_wait();
    const int64_t row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = kUpdateThreads >> 5;
    for (int g = blockIdx.y * n_warps + warp; g < groups; g += gridDim.y * n_warps) {
        const float* og = o + (row * groups + g) * G;
        float ss = 0.f;
        for (int j = lane; j < G; j += 32) ss = fmaf(og[j], og[j], ss);
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / static_cast<float>(G) + eps);
        for (int j = lane; j < G; j += 32) {
            const float z = to_float(gate[row * gate_stride + g * G + j]);
            out[(row * groups + g) * G + j] = from_float<T>(og[j] * inv * w[j] * (gate_act ? z : 1.f) * (1.f / (1.f + expf(-z))));
        }
    }
}

// src row t holds, from column col0 on, `heads` vectors of `width` elements; they land at
// pages[slot / page_size, head, slot % page_size, :].
template <typename T>
__global__ void write_rows_kernel(T* __restrict__ pages, const T* __restrict__ src, const int* __restrict__ slots,
                                  int row_stride, int col0, int heads, int width, int page_size, int64_t page_elems_total,
                                  int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int slot = slots[t];
    if (slot < 0) return;
    const int64_t page = slot / page_size, off = slot % page_size;
    const T* row = src + t * row_stride + col0;
    for (int i = threadIdx.x; i < heads * width; i += blockDim.x) {
        const int hd = i / width, e = i - hd * width;
        const int64_t at = ((page * heads + hd) * page_size + off) * width + e;
        if (at >= page_elems_total) { atomicExch(err, 2); return; }
        pages[at] = row[i];
    }
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_embed_positions(float* out, float* out2, const void* table, const void* pos_table, const int* tokens,
                                   const int* positions, int T, int D, int V, int P, float scale, int dtype, int* err_flag,
                                   cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0 || V <= 0 || (pos_table != nullptr && P <= 0)) return CVB_E_SIZE;
#define CALL(TY) launch_kernel(embed_positions_kernel<TY>, dim3(T), dim3(128), 0, stream, out, out2, (const TY*)table, \
                               (const TY*)pos_table, tokens, positions, D, V, P, scale, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_resid_update(float* h, const void* d1, const void* d2, const float* e, const float* vec, const float* w,
                                void* out, int T, int D, float eps, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0) return CVB_E_SIZE;
    if (d2 != nullptr && d1 == nullptr) return CVB_E_SHAPE;
    if (w != nullptr && out == nullptr) return CVB_E_SHAPE;
    auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec_ok = D % 4 == 0 && D <= kUpdateThreads * kUpdateChunks * 4 && al(h) && al(e) && al(vec) && al(w);
#define CALL(TY)                                                                                                          \
    if (vec_ok) launch_kernel(resid_update_vec_kernel<TY>, dim3(T), dim3(kUpdateThreads), 0, stream, h, (const TY*)d1,    \
                              (const TY*)d2, e, vec, w, (TY*)out, D, eps);                                                \
    else launch_kernel(resid_update_kernel<TY>, dim3(T), dim3(kUpdateThreads), 0, stream, h, (const TY*)d1, (const TY*)d2, \
                       e, vec, w, (TY*)out, D, eps)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_gelu_tanh(void* out, const void* x, int64_t n, int dtype, cudaStream_t stream) {
    if (n == 0) return CVB_OK;
    if (n < 0) return CVB_E_SIZE;
    if (dtype == CVB_DTYPE_BF16 && n % 8 == 0 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
        const int64_t chunks = n / 8, want8 = (chunks + 255) / 256;
        launch_kernel(gelu_tanh_bf16x8_kernel, dim3(static_cast<unsigned>(want8 < 148 * 16 ? want8 : 148 * 16)), dim3(256), 0, stream,
                      (__nv_bfloat16*)out, (const __nv_bfloat16*)x, chunks);
        return launch_status();
    }
    const int64_t want = (n + 255) / 256;
    const unsigned blocks = static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
#define CALL(TY) launch_kernel(gelu_tanh_kernel<TY>, dim3(blocks), dim3(256), 0, stream, (TY*)out, (const TY*)x, n)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_write_rows(void* pages, const void* src, const int* slots, int T, int row_stride, int col0, int heads,
                              int width, int page_size, int64_t page_elems_total, int dtype, int* err_flag,
                              cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || heads <= 0 || width <= 0 || page_size <= 0 || row_stride < col0 + heads * width || col0 < 0) return CVB_E_SIZE;
#define CALL(TY) launch_kernel(write_rows_kernel<TY>, dim3(T), dim3(128), 0, stream, (TY*)pages, (const TY*)src, slots, \
                               row_stride, col0, heads, width, page_size, page_elems_total, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_norm_add(float* h, const void* y, const float* bias, const float* w, void* copy, int T, int D, float eps,
                            int accumulate, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0) return CVB_E_SIZE;
    if (h == nullptr || y == nullptr || w == nullptr) return CVB_E_SHAPE;
    auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec_ok = D % 4 == 0 && D <= kUpdateThreads * kUpdateChunks * 4 && al(h) && al(bias) && al(w);
#define CALL(TY)                                                                                                              \
    if (vec_ok) launch_kernel(norm_add_vec_kernel<TY>, dim3(T), dim3(kUpdateThreads), 0, stream, h, (const TY*)y, bias, w,    \
                              (TY*)copy, D, eps, accumulate);                                                                 \
    else launch_kernel(norm_add_kernel<TY>, dim3(T), dim3(kUpdateThreads), 0, stream, h, (const TY*)y, bias, w, (TY*)copy,    \
                       D, eps, accumulate)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_bias_act(void* out, const void* x, const float* bias, int64_t n, int D, int act, int dtype, cudaStream_t stream) {
    if (n == 0) return CVB_OK;
    if (n < 0 || D <= 0 || act < 0 || act > 2) return CVB_E_SIZE;
    if (dtype == CVB_DTYPE_BF16 && D % 8 == 0 && n % 8 == 0 &&
        ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
        const int64_t chunks = n / 8, want8 = (chunks + 255) / 256;
        launch_kernel(bias_act_bf16x8_kernel, dim3(static_cast<unsigned>(want8 < 148 * 16 ? want8 : 148 * 16)), dim3(256), 0, stream,
                      (__nv_bfloat16*)out, (const __nv_bfloat16*)x, bias, chunks, D, act);
        return launch_status();
    }
    const int64_t want = (n + 255) / 256;
    const unsigned blocks = static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
#define CALL(TY) launch_kernel(bias_act_kernel<TY>, dim3(blocks), dim3(256), 0, stream, (TY*)out, (const TY*)x, bias, n, D, act)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_gated_norm(void* out, const float* o, const void* gate, int gate_stride, const float* w, int T, int groups, int G,
                              float eps, int gate_act, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || groups <= 0 || G <= 0 || gate_act < 0 || gate_act > 1) return CVB_E_SIZE;
    if (gate_stride < groups * G) return CVB_E_SHAPE;
    if (groups > 65535) return CVB_E_SIZE;
    const int per_block = kUpdateThreads / 32;
#define CALL(TY)                                                                                                                 \
    if (G > 256) launch_kernel(gated_norm_block_kernel<TY>, dim3(T, groups), dim3(kUpdateThreads), 0, stream, (TY*)out, o,       \
                               (const TY*)gate, gate_stride, w, groups, G, eps, gate_act);                                                 \
    else launch_kernel(gated_norm_kernel<TY>, dim3(T, (groups + per_block - 1) / per_block), dim3(kUpdateThreads), 0, stream,    \
                       (TY*)out, o, (const TY*)gate, gate_stride, w, groups, G, eps, gate_act)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}
