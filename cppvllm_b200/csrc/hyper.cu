// A residual stream of several copies ("streams") that sublayers read through learned weights and write back through a
// learned matrix, all in float32 under activations of any element type.
//
//   X [T, S, D] float: the S streams of every token.  A sublayer f with numbers a[S] (read), M[S, S] (from, to), b[S] (write)
//   and a norm with ONE weight g:
//       u = sum_s a_s x_s;   h = T( u / sqrt(mean(u^2) + eps) * g );   y = f(h);   x_t <- sum_s M[s, t] x_s + b_t y
//   (y may arrive as two addends that are summed in float: the routed experts' output and the shared expert's)
//   stream_embed : x_s = table[token] for every s
//   stream_step  : the write of one sublayer (optional) and the read and norm for the next (optional) in one pass: a block
//                  holds a token's row, forms the new streams from the old ones element by element (all S values of an
//                  element live in one thread, so the update is in place), stores them, and keeps the next sublayer's u in
//                  shared memory for the norm.  With a = 1 and no write it is the sum of the streams and the model's last norm.
// Sums run over s in rising order in float; the result of a token depends on nothing but its own row.
#include "common.cuh"

namespace cvb {

constexpr int kStreamThreads = 256;
constexpr int kMaxStreams = 8;

template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
stream_embed_kernel(float* __restrict__ X, const T* __restrict__ table, const int* __restrict__ tokens, int S, int D, int vocab,
                    int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int64_t t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicExch(err, 1);
        tok = 0;
    }
    const T* row = table + static_cast<int64_t>(tok) * D;
    float* out = X + t * S * D;
    for (int d = threadIdx.x; d < D; d += kStreamThreads) {
        const float v = to_float(row[d]);
        for (int s = 0; s < S; ++s) out[static_cast<int64_t>(s) * D + d] = v;
    }
}

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

// The same pass four elements at a time (D a multiple of 4) with the number of streams known to the compiler (1 to 4): 16-byte
// loads and stores of the streams, 8- or 16-byte ones of the sublayer's output and of the normed row, the weights in
// registers.  The order of every sum is that of the scalar form.
template <typename T, int NS>
__global__ void __launch_bounds__(kStreamThreads)
stream_step_vec_kernel(float* __restrict__ X, const T* __restrict__ y, const T* __restrict__ y2, const float* __restrict__ mix, const float* __restrict__ wout,
                       const float* __restrict__ win, const float* __restrict__ g, float eps, T* __restrict__ normed, int D) {
    pdl_trigger();
    extern __shared__ __align__(16) float smem[];
    float* us = smem;                                   // [D]
    float* scratch = smem + D;                          // [32]
    float m_r[NS][NS], b_r[NS], a_r[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
        b_r[s] = wout != nullptr ? wout[s] : 0.f;
        a_r[s] = win != nullptr ? win[s] : 1.f;
#pragma unroll
        for (int to = 0; to < NS; ++to) m_r[s][to] = mix != nullptr ? mix[s * NS + to] : 0.f;
    }
    const float gw = g != nullptr ? g[0] : 1.f;
    pdl_wait();
    const int64_t t = blockIdx.x;
    float* row = X + t * NS * D;
    float ss = 0.f;
    for (int d = threadIdx.x * 4; d < D; d += kStreamThreads * 4) {
        float4 x[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) x[s] = load4(row + static_cast<int64_t>(s) * D + d);
        if (y != nullptr) {
            float4 yv = load4(y + t * D + d);
            if (y2 != nullptr) { const float4 z = load4(y2 + t * D + d); yv.x += z.x; yv.y += z.y; yv.z += z.z; yv.w += z.w; }
            float4 nx[NS];
#pragma unroll
            for (int to = 0; to < NS; ++to) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    acc.x = fmaf(m_r[s][to], x[s].x, acc.x); acc.y = fmaf(m_r[s][to], x[s].y, acc.y);
                    acc.z = fmaf(m_r[s][to], x[s].z, acc.z); acc.w = fmaf(m_r[s][to], x[s].w, acc.w);
                }
                nx[to] = make_float4(fmaf(b_r[to], yv.x, acc.x), fmaf(b_r[to], yv.y, acc.y), fmaf(b_r[to], yv.z, acc.z), fmaf(b_r[to], yv.w, acc.w));
            }
#pragma unroll
            for (int s = 0; s < NS; ++s) { x[s] = nx[s]; store4(row + static_cast<int64_t>(s) * D + d, nx[s]); }
        }
        if (normed != nullptr) {
            float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                u.x = fmaf(a_r[s], x[s].x, u.x); u.y = fmaf(a_r[s], x[s].y, u.y); u.z = fmaf(a_r[s], x[s].z, u.z); u.w = fmaf(a_r[s], x[s].w, u.w);
            }
            ss = fmaf(u.x, u.x, ss); ss = fmaf(u.y, u.y, ss); ss = fmaf(u.z, u.z, ss); ss = fmaf(u.w, u.w, ss);
            store4(us + d, u);
        }
    }
    if (normed == nullptr) return;
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / static_cast<float>(D) + eps) * gw;
    for (int d = threadIdx.x * 4; d < D; d += kStreamThreads * 4) {
        const float4 u = load4(us + d);
        store4(normed + t * D + d, make_float4(u.x * inv, u.y * inv, u.z * inv, u.w * inv));
    }
}

template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
stream_step_kernel(float* __restrict__ X, const T* __restrict__ y, const T* __restrict__ y2, const float* __restrict__ mix, const float* __restrict__ wout,
                   const float* __restrict__ win, const float* __restrict__ g, float eps, T* __restrict__ normed, int S, int D) {
    pdl_trigger();
    extern __shared__ float smem[];
    float* us = smem;                                   // [D]: the next sublayer's input before its norm
    float* scratch = smem + D;                          // [32]
    __shared__ float m_s[kMaxStreams * kMaxStreams], b_s[kMaxStreams], a_s[kMaxStreams];
    if (threadIdx.x < S * S && mix != nullptr) m_s[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < S) {
        if (wout != nullptr) b_s[threadIdx.x] = wout[threadIdx.x];
        a_s[threadIdx.x] = win != nullptr ? win[threadIdx.x] : 1.f;
    }
    const float gw = g != nullptr ? g[0] : 1.f;
    pdl_wait();
    __syncthreads();
    const int64_t t = blockIdx.x;
    float* row = X + t * S * D;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += kStreamThreads) {
        float x[kMaxStreams];
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
            if (s < S) x[s] = row[static_cast<int64_t>(s) * D + d];
        if (y != nullptr) {
            const float yv = to_float(y[t * D + d]) + (y2 != nullptr ? to_float(y2[t * D + d]) : 0.f);
            float nx[kMaxStreams];
#pragma unroll
            for (int to = 0; to < kMaxStreams; ++to) {
                if (to >= S) break;
                float acc = 0.f;
#pragma unroll
                for (int s = 0; s < kMaxStreams; ++s)
                    if (s < S) acc = fmaf(m_s[s * S + to], x[s], acc);
                nx[to] = fmaf(b_s[to], yv, acc);
            }
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
                if (s < S) { x[s] = nx[s]; row[static_cast<int64_t>(s) * D + d] = nx[s]; }
        }
        if (normed != nullptr) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < kMaxStreams; ++s)
                if (s < S) u = fmaf(a_s[s], x[s], u);
            us[d] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (normed == nullptr) return;
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / static_cast<float>(D) + eps) * gw;
    for (int d = threadIdx.x; d < D; d += kStreamThreads) normed[t * D + d] = from_float<T>(us[d] * inv);
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_stream_embed(float* X, const void* table, const int* tokens, int T, int S, int D, int vocab, int dtype,
                                int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || S <= 0 || D <= 0 || vocab <= 0) return CVB_E_SIZE;
#define CALL(TY) launch_kernel(stream_embed_kernel<TY>, dim3(T), dim3(kStreamThreads), 0, stream, X, (const TY*)table, tokens, S, D, \
                               vocab, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
#undef VEC
    return launch_status();
}

// y, mix, wout: the write (all or none); y2: a second output added to y in float (a shared expert beside the routed ones).  normed: the read and norm (win and g optional: ones).
extern "C" int cvb_stream_step(float* X, const void* y, const void* y2, const float* mix, const float* wout, const float* win, const float* g,
                               float eps, void* normed, int T, int S, int D, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || S <= 0 || D <= 0) return CVB_E_SIZE;
    if (S > kMaxStreams) return CVB_E_UNSUPPORTED;
    if ((y != nullptr) != (mix != nullptr) || (y != nullptr) != (wout != nullptr)) return CVB_E_SHAPE;
    if ((y == nullptr && normed == nullptr) || (y2 != nullptr && y == nullptr)) return CVB_E_SHAPE;
    const size_t smem = (static_cast<size_t>(D) + 32) * sizeof(float);
    if (smem > 200 * 1024) return CVB_E_SIZE;
    const bool wide = D % 4 == 0 && ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(y2) | reinterpret_cast<uintptr_t>(normed)) & 15) == 0;
#define VEC(TY, NS)                                                                                                       \
    do {                                                                                                                  \
        if (smem > 48 * 1024)                                                                                             \
            cudaFuncSetAttribute(stream_step_vec_kernel<TY, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_kernel(stream_step_vec_kernel<TY, NS>, dim3(T), dim3(kStreamThreads), smem, stream, X, (const TY*)y, (const TY*)y2, mix, wout, win, g, \
                      eps, (TY*)normed, D);                                                                               \
    } while (0)
#define CALL(TY)                                                                                                          \
    do {                                                                                                                  \
        if (smem > 48 * 1024)                                                                                             \
            cudaFuncSetAttribute(stream_step_kernel<TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
        if (wide && S == 1) { VEC(TY, 1); }                                                                               \
        else if (wide && S == 2) { VEC(TY, 2); }                                                                          \
        else if (wide && S == 3) { VEC(TY, 3); }                                                                          \
        else if (wide && S == 4) { VEC(TY, 4); }                                                                          \
        else                                                                                                              \
        launch_kernel(stream_step_kernel<TY>, dim3(T), dim3(kStreamThreads), smem, stream, X, (const TY*)y, (const TY*)y2, mix, wout, win, g, eps, \
                      (TY*)normed, S, D);                                                                                 \
    } while (0)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
#undef VEC
    return launch_status();
}
