// A residual stream of several copies ("streams") that sublayers read through learned weights and write back through a
// learned matrix, all in float32 under activations of any element type.
//
//   X [T, S, D] float: the S streams of every token.  A sublayer f with numbers a[S] (read), M[S, S] (from, to), b[S] (write)
//   and a norm with ONE weight g:
//       u = sum_s a_s x_s;   h = T( u / sqrt(mean(u^2) + eps) * g );   y = f(h);   x_t <- sum_s M[s, t] x_s + b_t y
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

template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
stream_step_kernel(float* __restrict__ X, const T* __restrict__ y, const float* __restrict__ mix, const float* __restrict__ wout,
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
            const float yv = to_float(y[t * D + d]);
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
    return launch_status();
}

// y, mix, wout: the write (all or none).  normed: the read and norm (win and g optional: ones).
extern "C" int cvb_stream_step(float* X, const void* y, const float* mix, const float* wout, const float* win, const float* g,
                               float eps, void* normed, int T, int S, int D, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || S <= 0 || D <= 0) return CVB_E_SIZE;
    if (S > kMaxStreams) return CVB_E_UNSUPPORTED;
    if ((y != nullptr) != (mix != nullptr) || (y != nullptr) != (wout != nullptr)) return CVB_E_SHAPE;
    if (y == nullptr && normed == nullptr) return CVB_E_SHAPE;
    const size_t smem = (static_cast<size_t>(D) + 32) * sizeof(float);
    if (smem > 200 * 1024) return CVB_E_SIZE;
#define CALL(TY)                                                                                                          \
    do {                                                                                                                  \
        if (smem > 48 * 1024)                                                                                             \
            cudaFuncSetAttribute(stream_step_kernel<TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
        launch_kernel(stream_step_kernel<TY>, dim3(T), dim3(kStreamThreads), smem, stream, X, (const TY*)y, mix, wout, win, g, eps, \
                      (TY*)normed, S, D);                                                                                 \
    } while (0)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}
