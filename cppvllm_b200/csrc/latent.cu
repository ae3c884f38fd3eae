// What stands around attention over a cache of latent vectors (one vector per token, shared by all heads):
//
//   latent_prep      : per token, from the packed output of the down projections:
//                        cq = T( a / sqrt(mean(a^2) + eps) * wq )                 the query latent, normed
//                        c  = T( b / sqrt(mean(b^2) + eps) * wk )                 the key/value latent, normed
//                        kr = T( rot_p(r) )                                       the positional key part, turned by the token's position
//                      and [c | kr] written into the token's slot of the cache pages [page, slot in page, rank + rot].
//                      Either half may be left out (a layer that reads another layer's cache writes none).
//   latent_q_assemble: the query that the attention kernel reads, per token and head: [q_abs | rot_p(q_rot)], where q_abs
//                      (the unrotated query taken through the key up-projection, laid out [head, token, rank]) comes from a
//                      batched product and q_rot is the head's positional part inside the packed query projection.
//   head_gate        : att[t, h, :] = T( o[h, t, :] * sigmoid(g[t, h]) ): one gate per token and head, and the move from the
//                      batched product's [head, token, :] to rows of concatenated heads.  With `per_element` the gate has
//                      one number per element of the concatenated heads: att[t, i] = T( o[..] * sigmoid(g[t, i]) ).
//
// The rotation pairs element 2i with element 2i+1 of the first `rot` elements (cos and sin tables [positions, rot / 2],
// float); elements behind them pass unchanged.  Norm statistics and the rotation are float.
#include "common.cuh"

namespace cvb {

constexpr int kLatentThreads = 128;

template <typename T>
__device__ __forceinline__ void norm_part(T* __restrict__ out, const T* __restrict__ in, const float* __restrict__ w, int n,
                                          float eps, float* scratch) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += kLatentThreads) {
        const float v = to_float(in[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / static_cast<float>(n) + eps);
    for (int i = threadIdx.x; i < n; i += kLatentThreads) out[i] = from_float<T>(to_float(in[i]) * inv * w[i]);
}

// out[0 .. width): in[0 .. width) with the first `rot` elements turned by the angle tables' row.
template <typename T>
__device__ __forceinline__ void rotate_part(T* __restrict__ out, const T* __restrict__ in, const float* __restrict__ cs,
                                            const float* __restrict__ sn, int rot, int width) {
    for (int i = threadIdx.x; i < width; i += kLatentThreads) {
        float v = to_float(in[i]);
        if (i < rot) {
            const float c = cs[i >> 1], s = sn[i >> 1];
            const float other = to_float(in[i ^ 1]);
            v = (i & 1) ? v * c + other * s : v * c - other * s;
        }
        out[i] = from_float<T>(v);
    }
}

template <typename T>
__global__ void __launch_bounds__(kLatentThreads)
latent_prep_kernel(T* __restrict__ cq_out, T* __restrict__ pages, const T* __restrict__ packed, int stride, int q_off, int q_rank,
                   const float* __restrict__ wq, int kv_off, int rank, int rot_width, int rot, const float* __restrict__ wk,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, int max_pos, const int* __restrict__ positions,
                   const int* __restrict__ slots, int64_t total_slots, float eps, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int64_t t = blockIdx.x;
    const T* row = packed + t * stride;
    if (cq_out != nullptr) norm_part(cq_out + t * q_rank, row + q_off, wq, q_rank, eps, scratch);
    if (pages == nullptr) return;
    const int slot = slots[t];
    if (slot < 0) return;
    if (slot >= total_slots) {
        if (threadIdx.x == 0) atomicExch(err, 2);
        return;
    }
    int p = positions[t];
    if (p < 0 || p >= max_pos) {
        if (threadIdx.x == 0) atomicExch(err, 3);
        p = p < 0 ? 0 : max_pos - 1;
    }
    T* entry = pages + static_cast<int64_t>(slot) * (rank + rot_width);
    norm_part(entry, row + kv_off, wk, rank, eps, scratch);
    rotate_part(entry + rank, row + kv_off + rank, cos_t + static_cast<int64_t>(p) * (rot / 2), sin_t + static_cast<int64_t>(p) * (rot / 2),
                rot, rot_width);
}

template <typename T>
__global__ void __launch_bounds__(kLatentThreads)
latent_q_assemble_kernel(T* __restrict__ q_out, const T* __restrict__ q_abs, const T* __restrict__ q, int q_stride, int H, int nope,
                         int rank, int rot_width, int rot, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                         int max_pos, const int* __restrict__ positions, int T_total, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int h = blockIdx.y;
    int p = positions[t];
    if (p < 0 || p >= max_pos) {
        if (threadIdx.x == 0) atomicExch(err, 3);
        p = p < 0 ? 0 : max_pos - 1;
    }
    T* dst = q_out + (t * H + h) * (rank + rot_width);
    const T* src = q_abs + (static_cast<int64_t>(h) * T_total + t) * rank;
    for (int i = threadIdx.x; i < rank; i += kLatentThreads) dst[i] = src[i];
    rotate_part(dst + rank, q + t * q_stride + h * (nope + rot_width) + nope, cos_t + static_cast<int64_t>(p) * (rot / 2),
                sin_t + static_cast<int64_t>(p) * (rot / 2), rot, rot_width);
}

template <typename T>
__global__ void __launch_bounds__(kLatentThreads)
head_gate_kernel(T* __restrict__ out, const T* __restrict__ o, const T* __restrict__ gate, int gate_stride, int H, int vd, int T_total,
                 int per_element) {
    pdl_trigger();
    pdl_wait();
    const int64_t t = blockIdx.x;
    for (int i = blockIdx.y * kLatentThreads + threadIdx.x; i < H * vd; i += gridDim.y * kLatentThreads) {
        const int h = i / vd, j = i - h * vd;
        const float z = to_float(gate[t * gate_stride + (per_element ? i : h)]);
        out[t * H * vd + i] = from_float<T>(to_float(o[(static_cast<int64_t>(h) * T_total + t) * vd + j]) * (1.f / (1.f + expf(-z))));
    }
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_latent_prep(void* cq_out, void* pages, const void* packed, int T, int stride, int q_off, int q_rank, const float* wq,
                               int kv_off, int rank, int rot_width, int rot, const float* wk, const float* cos_t, const float* sin_t,
                               int max_pos, const int* positions, const int* slots, int64_t total_slots, float eps, int dtype,
                               int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || stride <= 0) return CVB_E_SIZE;
    if (cq_out != nullptr && (q_rank <= 0 || q_off < 0 || q_off + q_rank > stride || wq == nullptr)) return CVB_E_SHAPE;
    if (pages != nullptr && (rank <= 0 || rot_width < 0 || rot < 0 || rot > rot_width || rot % 2 || kv_off < 0 ||
                             kv_off + rank + rot_width > stride || wk == nullptr || (rot > 0 && (cos_t == nullptr || sin_t == nullptr)) ||
                             max_pos <= 0 || total_slots <= 0))
        return CVB_E_SHAPE;
#define CALL(TY) launch_kernel(latent_prep_kernel<TY>, dim3(T), dim3(kLatentThreads), 0, stream, (TY*)cq_out, (TY*)pages, \
                               (const TY*)packed, stride, q_off, q_rank, wq, kv_off, rank, rot_width, rot, wk, cos_t, sin_t, max_pos, \
                               positions, slots, total_slots, eps, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_latent_q_assemble(void* q_out, const void* q_abs, const void* q, int T, int q_stride, int H, int nope, int rank,
                                     int rot_width, int rot, const float* cos_t, const float* sin_t, int max_pos, const int* positions,
                                     int dtype, int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || H <= 0 || H > 65535 || nope <= 0 || rank <= 0 || rot_width < 0 || max_pos <= 0) return CVB_E_SIZE;
    if (rot < 0 || rot > rot_width || rot % 2 || q_stride < H * (nope + rot_width)) return CVB_E_SHAPE;
#define CALL(TY) launch_kernel(latent_q_assemble_kernel<TY>, dim3(T, H), dim3(kLatentThreads), 0, stream, (TY*)q_out, (const TY*)q_abs, \
                               (const TY*)q, q_stride, H, nope, rank, rot_width, rot, cos_t, sin_t, max_pos, positions, T, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_head_gate(void* out, const void* o, const void* gate, int T, int gate_stride, int H, int vd, int per_element,
                             int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || H <= 0 || vd <= 0 || gate_stride < (per_element ? H * vd : H)) return CVB_E_SIZE;
    const int per_row = (H * vd + kLatentThreads - 1) / kLatentThreads;
#define CALL(TY) launch_kernel(head_gate_kernel<TY>, dim3(T, per_row < 64 ? per_row : 64), dim3(kLatentThreads), 0, stream, (TY*)out, (const TY*)o, (const TY*)gate, \
                               gate_stride, H, vd, T, per_element)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}
