// What stands around the sublayers of a layer whose sublayers are wrapped twice (a norm in front, a norm behind), read their
// input through a short causal convolution and leave through a learned gate; and what stands around attention with a norm
// over the whole query and key projections.  The residual stream is float; T is the activations' element type.
//
//   input_conv      : out[t, c] = T( a[t, c] + sum_j w[j, c] * a[t - K + 1 + j, c] ): a causal convolution over time on each
//                     channel, added to its own input (w holds one row of D weights per tap, the oldest tap first).  Tokens before the portion come from the request's history (the last
//                     K - 1 inputs of its earlier portions, zero at admission), which lies in the request's state row.
//   gated_norm_add  : v = y * sigmoid(z + b);  h[t, :] += v / sqrt(mean(v^2) + eps) * w   (the sublayer's output through its gate,
//                     the norm behind the sublayer, the sum into the stream: one kernel).  With a second weight w2 it also
//                     leaves out2[t, :] = T( h / sqrt(mean(h^2) + eps2) * w2 ), the norm in front of the next sublayer, while the
//                     new row is still on the chip.  With a history it also replaces the request's convolution history by the
//                     last K - 1 rows of `a` (the block of a request's first token does that; the convolution that read the
//                     history ran in an earlier kernel).
//   glu_clamped     : g = min(gu[t, i], L), u = clamp(gu[t, I + i], -L, L);  out = T( g * sigmoid(alpha g) * (u + 1) )
//   add_gated_rows  : y[t, :] = T( y[t, :] + sigmoid(z[t]) * s[t, :] )   (a shared expert joins the routed ones through one
//                     gate per token)
//   wide_qk_prep    : q[t, :] = T( q / sqrt(mean(q^2) + eps) * wq * (1 + coef * ln(floor((p + 1) / every) + 1)) ) over the WHOLE
//                     query projection (all heads at once), k likewise with wk and no temperature; k and v land in the cache
//                     pages [page, kv head, slot in page, dk + dv] (a head's key, then its value).
#include "common.cuh"

namespace cvb {

constexpr int kSandThreads = 256;

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(kSandThreads)
input_conv_kernel(T* __restrict__ out, const T* __restrict__ a, const float* __restrict__ w, int D, int taps,
                  const float* __restrict__ state, int64_t state_floats, int64_t hist_off, const int* __restrict__ seq_of_token,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, int num_slots, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int s = seq_of_token[t];
    const int local = static_cast<int>(t) - cu_seqlens[s];
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0) atomicExch(err, 2);
        return;
    }
    const float* hist = state + static_cast<int64_t>(slot) * state_floats + hist_off;
    for (int c = threadIdx.x; c < D; c += kSandThreads) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int o = local - (taps - 1) + j;
            const float x = o >= 0 ? to_float(a[(t - (taps - 1) + j) * D + c]) : hist[static_cast<int64_t>(local + j) * D + c];
            acc = fmaf(w[static_cast<int64_t>(j) * D + c], x, acc);
        }
        out[t * D + c] = from_float<T>(to_float(a[t * D + c]) + acc);
    }
}

// the same with 16 bytes of a row per thread (D a multiple of the chunk, rows on 16-byte boundaries); a channel's sum runs over
// the taps in the same order as above
template <typename T>
__global__ void __launch_bounds__(kSandThreads)
input_conv_vec_kernel(T* __restrict__ out, const T* __restrict__ a, const float* __restrict__ w, int D, int taps,
                      const float* __restrict__ state, int64_t state_floats, int64_t hist_off, const int* __restrict__ seq_of_token,
                      const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, int num_slots, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    constexpr int N = 16 / sizeof(T);
    const int64_t t = blockIdx.x;
    const int s = seq_of_token[t];
    const int local = static_cast<int>(t) - cu_seqlens[s];
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0) atomicExch(err, 2);
        return;
    }
    const float* hist = state + static_cast<int64_t>(slot) * state_floats + hist_off;
    for (int c = threadIdx.x * N; c < D; c += kSandThreads * N) {
        float acc[N], x[N];
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int o = local - (taps - 1) + j;
            if (o >= 0) {
                alignas(16) T v[N];
                *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(a + (t - (taps - 1) + j) * D + c);
#pragma unroll
                for (int i = 0; i < N; ++i) x[i] = to_float(v[i]);
            } else {
                const float* hp = hist + static_cast<int64_t>(local + j) * D + c;
#pragma unroll
                for (int i = 0; i < N; ++i) x[i] = hp[i];
            }
            alignas(16) float wj[N];
#pragma unroll
            for (int i = 0; i < N; i += 4)
                *reinterpret_cast<float4*>(wj + i) = *reinterpret_cast<const float4*>(w + static_cast<int64_t>(j) * D + c + i);
#pragma unroll
            for (int i = 0; i < N; ++i) acc[i] = fmaf(wj[i], x[i], acc[i]);
        }
        alignas(16) T y[N];                               // x holds the token's own row: the last tap's
#pragma unroll
        for (int i = 0; i < N; ++i) y[i] = from_float<T>(x[i] + acc[i]);
        *reinterpret_cast<uint4*>(out + t * D + c) = *reinterpret_cast<const uint4*>(y);
    }
}

template <typename T>
__global__ void __launch_bounds__(kSandThreads)
gated_norm_add_kernel(float* __restrict__ h, const T* __restrict__ y, const T* __restrict__ z, const float* __restrict__ zb,
                      const float* __restrict__ w, float eps, const float* __restrict__ w2, float eps2, T* __restrict__ out2, int D,
                      const T* __restrict__ a, float* __restrict__ state, int64_t state_floats, int64_t hist_off, int taps,
                      const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                      int num_slots) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float row[];                  // [D]
    __shared__ float scratch[32];
    const int64_t t = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += kSandThreads) {
        float v = to_float(y[t * D + i]);
        if (z) v *= sigmoid_f(to_float(z[t * D + i]) + (zb ? zb[i] : 0.f));
        row[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / static_cast<float>(D) + eps);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < D; i += kSandThreads) {
        const float r = h[t * D + i] + row[i] * inv * w[i];
        h[t * D + i] = r;
        row[i] = r;
        ss2 = fmaf(r, r, ss2);
    }
    if (w2 != nullptr) {
        ss2 = block_sum(ss2, scratch);
        const float inv2 = 1.f / sqrtf(ss2 / static_cast<float>(D) + eps2);
        for (int i = threadIdx.x; i < D; i += kSandThreads) out2[t * D + i] = from_float<T>(row[i] * inv2 * w2[i]);
    }
    if (a != nullptr && taps > 1) {
        const int s = seq_of_token[t];
        const int begin = cu_seqlens[s];
        if (static_cast<int>(t) != begin) return;
        const int n = cu_seqlens[s + 1] - begin;
        const int slot = state_slots[s];
        if (slot < 0 || slot >= num_slots) return;          // reported by the convolution in front
        float* hist = state + static_cast<int64_t>(slot) * state_floats + hist_off;
        // a thread owns a channel and walks its history from the oldest entry on: an entry is read before it is overwritten
        for (int c = threadIdx.x; c < D; c += kSandThreads) {
            for (int m = 0; m < taps - 1; ++m) {
                const int o = n - (taps - 1) + m;
                hist[static_cast<int64_t>(m) * D + c] = o >= 0 ? to_float(a[static_cast<int64_t>(begin + o) * D + c])
                                                               : hist[static_cast<int64_t>(n + m) * D + c];
            }
        }
    }
}

template <typename T>
__global__ void glu_clamped_kernel(T* __restrict__ out, const T* __restrict__ gu, int64_t n, int I, float limit, float alpha) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = i / I;
        const int c = static_cast<int>(i - t * I);
        const float g = fminf(to_float(gu[t * 2 * I + c]), limit);
        const float u = fminf(fmaxf(to_float(gu[t * 2 * I + I + c]), -limit), limit);
        out[i] = from_float<T>(g * sigmoid_f(alpha * g) * (u + 1.f));
    }
}

// 16 bytes of gate and of up per thread: I is a multiple of the chunk and all rows start on 16 bytes
template <typename T>
__global__ void glu_clamped_vec_kernel(T* __restrict__ out, const T* __restrict__ gu, int64_t n_chunks, int I, float limit, float alpha) {
    pdl_trigger();
    pdl_wait();
    constexpr int N = 16 / sizeof(T);
    const int64_t k = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (k >= n_chunks) return;
    const int per_row = I / N;
    const int64_t t = k / per_row;
    const int c = static_cast<int>(k - t * per_row) * N;
    alignas(16) T g[N], u[N], o[N];
    *reinterpret_cast<uint4*>(g) = *reinterpret_cast<const uint4*>(gu + t * 2 * I + c);
    *reinterpret_cast<uint4*>(u) = *reinterpret_cast<const uint4*>(gu + t * 2 * I + I + c);
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const float gi = fminf(to_float(g[i]), limit);
        const float ui = fminf(fmaxf(to_float(u[i]), -limit), limit);
        o[i] = from_float<T>(gi * sigmoid_f(alpha * gi) * (ui + 1.f));
    }
    *reinterpret_cast<uint4*>(out + t * I + c) = *reinterpret_cast<const uint4*>(o);
}

template <typename T>
__global__ void add_gated_rows_kernel(T* __restrict__ y, const T* __restrict__ s, const float* __restrict__ z, int z_stride, int64_t n,
                                      int D) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = i / D;
        y[i] = from_float<T>(to_float(y[i]) + sigmoid_f(z[t * z_stride]) * to_float(s[i]));
    }
}

// One block per token.  The packed row holds the query projection from column 0 and, when `nk` > 0, the key projection from
// column nq and the value projection from column nq + nk on (KV heads of dk, then KV heads of dv).
template <typename T>
__global__ void __launch_bounds__(kSandThreads)
wide_qk_prep_kernel(T* __restrict__ q_out, T* __restrict__ pages, const T* __restrict__ packed, int stride, const float* __restrict__ wq,
                    const float* __restrict__ wk, const int* __restrict__ positions, const int* __restrict__ slots, int nq, int KV,
                    int dk, int dv, int page_size, int64_t num_pages, float eps, float temp_coef, int temp_every, int write_kv,
                    int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int64_t t = blockIdx.x;
    const T* row = packed + t * stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < nq; i += kSandThreads) { const float v = to_float(row[i]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    const int p = positions[t];
    const float temp = temp_every > 0 ? 1.f + temp_coef * logf(static_cast<float>((p + 1) / temp_every + 1)) : 1.f;
    const float inv = temp / sqrtf(ss / static_cast<float>(nq) + eps);
    for (int i = threadIdx.x; i < nq; i += kSandThreads) q_out[t * nq + i] = from_float<T>(to_float(row[i]) * wq[i] * inv);
    if (!write_kv) return;
    const int nk = KV * dk, nv = KV * dv;
    float sk = 0.f;
    for (int i = threadIdx.x; i < nk; i += kSandThreads) { const float v = to_float(row[nq + i]); sk = fmaf(v, v, sk); }
    sk = block_sum(sk, scratch);
    const float invk = 1.f / sqrtf(sk / static_cast<float>(nk) + eps);
    const int slot = slots[t];
    const int64_t page = slot / page_size;
    if (slot < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicExch(err, 3);
        return;
    }
    const int off = slot - static_cast<int>(page) * page_size;
    const int ew = dk + dv;
    for (int i = threadIdx.x; i < nk; i += kSandThreads) {
        const int g = i / dk, e = i - g * dk;
        pages[((page * KV + g) * page_size + off) * ew + e] = from_float<T>(to_float(row[nq + i]) * wk[i] * invk);
    }
    for (int i = threadIdx.x; i < nv; i += kSandThreads) {
        const int g = i / dv, e = i - g * dv;
        pages[((page * KV + g) * page_size + off) * ew + dk + e] = row[nq + nk + i];
    }
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_input_conv(void* out, const void* a, const float* w, int T, int D, int taps, const float* state, int64_t state_floats,
                              int64_t hist_off, const int* seq_of_token, const int* cu_seqlens, const int* state_slots, int num_slots,
                              int dtype, int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0 || taps <= 0 || num_slots <= 0) return CVB_E_SIZE;
    if (hist_off < 0 || state_floats < hist_off + static_cast<int64_t>(taps - 1) * D) return CVB_E_SHAPE;
    const bool aligned = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
#define CALL(TY)                                                                                                                          \
    if (aligned && D % (16 / (int)sizeof(TY)) == 0)                                                                                       \
        launch_kernel(input_conv_vec_kernel<TY>, dim3(T), dim3(kSandThreads), 0, stream, (TY*)out, (const TY*)a, w, D, taps, state,       \
                      state_floats, hist_off, seq_of_token, cu_seqlens, state_slots, num_slots, err_flag);                                \
    else                                                                                                                                  \
        launch_kernel(input_conv_kernel<TY>, dim3(T), dim3(kSandThreads), 0, stream, (TY*)out, (const TY*)a, w, D, taps, state,           \
                      state_floats, hist_off, seq_of_token, cu_seqlens, state_slots, num_slots, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_gated_norm_add(float* h, const void* y, const void* z, const float* zb, const float* w, float eps, const float* w2,
                                  float eps2, void* out2, int T, int D, const void* a, float* state, int64_t state_floats,
                                  int64_t hist_off, int taps, const int* seq_of_token, const int* cu_seqlens, const int* state_slots,
                                  int num_slots, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0 || D > 12288) return CVB_E_SIZE;
    if (h == nullptr || y == nullptr || w == nullptr || (w2 != nullptr && out2 == nullptr)) return CVB_E_SHAPE;
    if (a != nullptr && taps > 1 &&
        (state == nullptr || hist_off < 0 || state_floats < hist_off + static_cast<int64_t>(taps - 1) * D || num_slots <= 0))
        return CVB_E_SHAPE;
#define CALL(TY) launch_kernel(gated_norm_add_kernel<TY>, dim3(T), dim3(kSandThreads), static_cast<size_t>(D) * sizeof(float), stream, h, \
                               (const TY*)y, (const TY*)z, zb, w, eps, w2, eps2, (TY*)out2, D, (const TY*)a, state, state_floats,       \
                               hist_off, taps, seq_of_token, cu_seqlens, state_slots, num_slots)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_glu_clamped(void* out, const void* gate_up, int T, int I, float limit, float alpha, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || I <= 0) return CVB_E_SIZE;
    const int64_t n = static_cast<int64_t>(T) * I, want = (n + 255) / 256;
    const unsigned blocks = static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
    const bool aligned = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(gate_up)) & 15) == 0;
#define CALL(TY)                                                                                                                          \
    if (aligned && I % (16 / (int)sizeof(TY)) == 0) {                                                                                     \
        const int64_t nc = n / (16 / (int)sizeof(TY));                                                                                    \
        launch_kernel(glu_clamped_vec_kernel<TY>, dim3(static_cast<unsigned>((nc + 255) / 256)), dim3(256), 0, stream, (TY*)out,          \
                      (const TY*)gate_up, nc, I, limit, alpha);                                                                           \
    } else                                                                                                                                \
        launch_kernel(glu_clamped_kernel<TY>, dim3(blocks), dim3(256), 0, stream, (TY*)out, (const TY*)gate_up, n, I, limit, alpha)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_add_gated_rows(void* y, const void* s, const float* z, int z_stride, int T, int D, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0 || z_stride <= 0) return CVB_E_SIZE;
    const int64_t n = static_cast<int64_t>(T) * D, want = (n + 255) / 256;
    const unsigned blocks = static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
#define CALL(TY) launch_kernel(add_gated_rows_kernel<TY>, dim3(blocks), dim3(256), 0, stream, (TY*)y, (const TY*)s, z, z_stride, n, D)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_wide_qk_prep(void* q_out, void* pages, const void* packed, int T, int stride, const float* wq, const float* wk,
                                const int* positions, const int* slots, int nq, int KV, int dk, int dv, int page_size,
                                int64_t num_pages, float eps, float temp_coef, int temp_every, int write_kv, int dtype, int* err_flag,
                                cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || nq <= 0 || KV <= 0 || dk <= 0 || dv <= 0 || page_size <= 0) return CVB_E_SIZE;
    if (stride < nq + (write_kv ? KV * (dk + dv) : 0) || temp_every < 0) return CVB_E_SHAPE;
    if (write_kv && (pages == nullptr || wk == nullptr || slots == nullptr || num_pages <= 0)) return CVB_E_SHAPE;
#define CALL(TY) launch_kernel(wide_qk_prep_kernel<TY>, dim3(T), dim3(kSandThreads), 0, stream, (TY*)q_out, (TY*)pages, (const TY*)packed, \
                               stride, wq, wk, positions, slots, nq, KV, dk, dv, page_size, num_pages, eps, temp_coef, temp_every,      \
                               write_kv, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}
