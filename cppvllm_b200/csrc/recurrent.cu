// Mixers that carry a matrix of fixed size per request and head from token to token instead of a cache that grows:
//
//   lightning_prep : q = silu(a_q), k = silu(a_k), v = silu(a_v) in float, from a packed projection
//   lightning_scan : S <- d_h S + k v^T;  o = S^T q
//   delta_prep     : per token, everything the delta rule needs, in float: short causal convolutions over time (per channel,
//                    the last tap on the current token, history from the request's state where the portion begins) with
//                    silu behind them; q and k made unit vectors per head (x / sqrt(sum x^2 + 1e-6); q also times
//                    dk^-1/2); b = sigmoid(.); the decay g = exp(-exp(A_h) softplus(a + dt)) per head and key channel
//   conv_history   : the last taps - 1 raw inputs of every request's portion become the history of its next one
//   delta_scan     : S <- diag(g) S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q      (query/key head h / (H / G))
//                    The decay is one number per head and key channel, or (`gd` = 1) one number per head: S <- g S.
//
// S is [dk, dv] per (request, head), float, in the request's state slot; portions of any length continue where the
// state stands, one token after the other in the same order of operations, so cutting a sequence changes no bit.
// A block owns 16 columns of S of one (request, head); eight lanes share a column and add their parts up by shuffles.  The
// tokens of a portion travel through two stages of shared memory by cp.async.
#include "common.cuh"
#include "sm100.cuh"

namespace cvb {

constexpr int kScanThreads = 128;
constexpr int kScanLanes = 8;                            // lanes that share a column of S
constexpr int kScanCols = kScanThreads / kScanLanes;     // columns of S per block
constexpr int kScanChunk = 8;                            // tokens per stage

__device__ __forceinline__ float silu_of(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_of(float z) { return 1.f / (1.f + expf(-z)); }

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(smem)), "l"(gmem));
}

// q = silu(a_q), k = silu(a_k), v = silu(a_v) in float, from the column ranges of a packed projection.
template <typename T>
__global__ void lightning_prep_kernel(float* __restrict__ qf, float* __restrict__ kf, float* __restrict__ vf, const T* __restrict__ packed,
                                      int stride, int q_off, int k_off, int v_off, int nqk, int nv, int64_t total) {
    pdl_trigger();
    pdl_wait();
    const int per = 2 * nqk + nv;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = i / per;
        const int c = static_cast<int>(i - t * per);
        const T* row = packed + t * stride;
        if (c < nqk) qf[t * nqk + c] = silu_of(to_float(row[q_off + c]));
        else if (c < 2 * nqk) kf[t * nqk + c - nqk] = silu_of(to_float(row[k_off + c - nqk]));
        else vf[t * nv + c - 2 * nqk] = silu_of(to_float(row[v_off + c - 2 * nqk]));
    }
}

// The scan of both rules.  A block owns kScanCols columns of S of one (request, head); kScanLanes lanes share a column
// (rows r * kScanLanes + lane part) and add their parts up by shuffles.  The tokens' q, k (and g), v (and b) travel through
// two stages of shared memory by cp.async, kScanChunk tokens a stage, so that the next tokens arrive while these are used.
// MODE 1: S <- diag(g) S; u = b (v - S^T k); S <- S + k u^T; o = S^T q.  MODE 2: the same with one decay per head and token
// (S <- g S).  MODE 0: S <- d S + k v^T; o = S^T q.
template <int KPT, int MODE>
__global__ void __launch_bounds__(kScanThreads)
recurrent_scan_kernel(float* __restrict__ out, const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vv,
                      const float* __restrict__ gg, const float* __restrict__ bb, const float* __restrict__ decay,
                      float* __restrict__ state, int64_t state_floats, const int* __restrict__ cu_seqlens,
                      const int* __restrict__ state_slots, int num_slots, int H, int G, int dk, int dv, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr int dkp = KPT * kScanLanes;
    constexpr bool DELTA = MODE != 0;
    constexpr int kArrays = MODE == 1 ? 3 : 2;
    constexpr int kStage = kArrays * kScanChunk * dkp + kScanChunk * kScanCols + 2 * kScanChunk;
    const int s = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * kScanCols;
    const int kvh = h / (H / G);
    const int tid = threadIdx.x, col = tid / kScanLanes, part = tid % kScanLanes, j = j0 + col;
    const int begin = cu_seqlens[s], end = cu_seqlens[s + 1];
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (tid == 0) atomicExch(err, 2);
        return;
    }
    for (int i = tid; i < 2 * kStage; i += kScanThreads) sm[i] = 0.f;       // the rows past dk stay zero for good
    __syncthreads();
    float* st = state + static_cast<int64_t>(slot) * state_floats + static_cast<int64_t>(h) * dk * dv;
    float S[KPT];
#pragma unroll
    for (int r = 0; r < KPT; ++r) {
        const int i = r * kScanLanes + part;
        S[r] = (i < dk && j < dv) ? st[static_cast<int64_t>(i) * dv + j] : 0.f;
    }
    const float d = DELTA ? 1.f : decay[h];
    const bool vec = (dk & 3) == 0 && (dv & 3) == 0;

    auto load = [&](int t0, int stage) {
        const int n = min(kScanChunk, end - t0);
        float* qs = sm + stage * kStage;
        float* ks = qs + kScanChunk * dkp;
        float* gs = ks + kScanChunk * dkp;                                  // MODE 1 only
        float* vs = qs + kArrays * kScanChunk * dkp;
        float* bs = vs + kScanChunk * kScanCols;
        float* g1 = bs + kScanChunk;                                        // MODE 2 only: one decay per token
        if (vec) {
            const int dk4 = dk >> 2;
            for (int idx = tid; idx < n * dk4; idx += kScanThreads) {
                const int tt = idx / dk4, i = (idx - tt * dk4) * 4;
                const int64_t tok = t0 + tt;
                cp_async16(qs + tt * dkp + i, qn + (tok * G + kvh) * dk + i, true);
                cp_async16(ks + tt * dkp + i, kn + (tok * G + kvh) * dk + i, true);
                if (MODE == 1) cp_async16(gs + tt * dkp + i, gg + (tok * H + h) * dk + i, true);
            }
            for (int idx = tid; idx < n * (kScanCols / 4); idx += kScanThreads) {
                const int tt = idx / (kScanCols / 4), c = (idx - tt * (kScanCols / 4)) * 4;
                if (j0 + c < dv) cp_async16(vs + tt * kScanCols + c, vv + (static_cast<int64_t>(t0 + tt) * H + h) * dv + j0 + c, true);
            }
        } else {
            for (int idx = tid; idx < n * dk; idx += kScanThreads) {
                const int tt = idx / dk, i = idx - tt * dk;
                const int64_t tok = t0 + tt;
                cp_async4(qs + tt * dkp + i, qn + (tok * G + kvh) * dk + i);
                cp_async4(ks + tt * dkp + i, kn + (tok * G + kvh) * dk + i);
                if (MODE == 1) cp_async4(gs + tt * dkp + i, gg + (tok * H + h) * dk + i);
            }
            for (int idx = tid; idx < n * kScanCols; idx += kScanThreads) {
                const int tt = idx / kScanCols, c = idx - tt * kScanCols;
                if (j0 + c < dv) cp_async4(vs + tt * kScanCols + c, vv + (static_cast<int64_t>(t0 + tt) * H + h) * dv + j0 + c);
            }
        }
        if (DELTA && tid < n) cp_async4(bs + tid, bb + static_cast<int64_t>(t0 + tid) * H + h);
        if (MODE == 2 && tid < n) cp_async4(g1 + tid, gg + static_cast<int64_t>(t0 + tid) * H + h);
    };

    if (begin < end) load(begin, 0);
    cp_async_commit();
    int stage = 0;
    for (int t0 = begin; t0 < end; t0 += kScanChunk, stage ^= 1) {
        const int n = min(kScanChunk, end - t0);
        if (t0 + kScanChunk < end) load(t0 + kScanChunk, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();                                                  // everything but the newest group: this stage
        __syncthreads();
        const float* qs = sm + stage * kStage;
        const float* ks = qs + kScanChunk * dkp;
        const float* gs = ks + kScanChunk * dkp;
        const float* vs = qs + kArrays * kScanChunk * dkp;
        const float* bs = vs + kScanChunk * kScanCols;
        const float* g1 = bs + kScanChunk;
        auto token = [&](int tt) {
            const float* kq = ks + tt * dkp + part;
            const float* qq = qs + tt * dkp + part;
            const float v = vs[tt * kScanCols + col];
            float o0 = 0.f, o1 = 0.f;
            if (DELTA) {
                const float* gq = gs + tt * dkp + part;
                const float gh = MODE == 2 ? g1[tt] : 1.f;
                float d0 = 0.f, d1 = 0.f;
#pragma unroll
                for (int r = 0; r < KPT; ++r) {
                    S[r] *= MODE == 2 ? gh : gq[r * kScanLanes];
                    if (r & 1) d1 = fmaf(S[r], kq[r * kScanLanes], d1); else d0 = fmaf(S[r], kq[r * kScanLanes], d0);
                }
                float dot = d0 + d1;
#pragma unroll
                for (int m = 1; m < kScanLanes; m <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, m);
                const float u = bs[tt] * (v - dot);
#pragma unroll
                for (int r = 0; r < KPT; ++r) {
                    S[r] = fmaf(kq[r * kScanLanes], u, S[r]);
                    if (r & 1) o1 = fmaf(S[r], qq[r * kScanLanes], o1); else o0 = fmaf(S[r], qq[r * kScanLanes], o0);
                }
            } else {
#pragma unroll
                for (int r = 0; r < KPT; ++r) {
                    S[r] = fmaf(d, S[r], kq[r * kScanLanes] * v);
                    if (r & 1) o1 = fmaf(S[r], qq[r * kScanLanes], o1); else o0 = fmaf(S[r], qq[r * kScanLanes], o0);
                }
            }
            float o = o0 + o1;
#pragma unroll
            for (int m = 1; m < kScanLanes; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
            if (part == 0 && j < dv) out[(static_cast<int64_t>(t0 + tt) * H + h) * dv + j] = o;
        };
        if (n == kScanChunk) {                                               // unrolled: the tokens' shuffles and loads overlap
#pragma unroll
            for (int tt = 0; tt < kScanChunk; ++tt) token(tt);
        } else {
            for (int tt = 0; tt < n; ++tt) token(tt);
        }
        __syncthreads();                                                     // the stage may be filled again
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < KPT; ++r) {
        const int i = r * kScanLanes + part;
        if (i < dk && j < dv) st[static_cast<int64_t>(i) * dv + j] = S[r];
    }
}

// One block per token.  Channels: q [G * dk], k [G * dk], v [H * dv], in this order both in the packed row (from
// column qkv_off on) and in the convolution weights [C, taps] and the history [taps - 1, C] (oldest first).
constexpr int kPrepThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kPrepThreads)
delta_prep_kernel(float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vv, float* __restrict__ gg, float* __restrict__ bb,
                  const T* __restrict__ packed, int stride, int qkv_off, const float* __restrict__ conv_w, int taps,
                  const float* __restrict__ a, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                  const float* __restrict__ b, const float* __restrict__ state, int64_t state_floats, int64_t conv_off,
                  const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                  int num_slots, int H, int G, int dk, int dv, int gd, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];                 // conv outputs of q and k: [2 * G * dk]
    const int64_t t = blockIdx.x;
    const int tid = threadIdx.x;
    const int s = seq_of_token[t];
    const int local = static_cast<int>(t) - cu_seqlens[s];
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (tid == 0) atomicExch(err, 2);
        return;
    }
    const int QK = G * dk, C = 2 * QK + H * dv;
    const float* hist = state + static_cast<int64_t>(slot) * state_floats + conv_off;
    for (int c = tid; c < C; c += kPrepThreads) {
        float acc = 0.f;
        for (int jt = 0; jt < taps; ++jt) {
            const int o = local - (taps - 1) + jt;          // which token of the portion this tap reads; negative: before it
            const float x = o >= 0 ? to_float(packed[(t - (taps - 1) + jt) * stride + qkv_off + c])
                                   : hist[static_cast<int64_t>(local + jt) * C + c];
            acc = fmaf(conv_w[static_cast<int64_t>(c) * taps + jt], x, acc);
        }
        const float y = silu_of(acc);
        if (c < 2 * QK) sm[c] = y;
        else vv[t * H * dv + (c - 2 * QK)] = y;
    }
    __syncthreads();
    const int warp = tid >> 5, lane = tid & 31;
    for (int grp = warp; grp < 2 * G; grp += kPrepThreads / 32) {
        const float* x = sm + grp * dk;
        float ss = 0.f;
        for (int i = lane; i < dk; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        float inv = 1.f / sqrtf(ss + 1e-6f);
        float* dst;
        if (grp < G) { inv *= 1.f / sqrtf(static_cast<float>(dk)); dst = qn + (t * G + grp) * dk; }
        else dst = kn + (t * G + (grp - G)) * dk;
        for (int i = lane; i < dk; i += 32) dst[i] = x[i] * inv;
    }
    for (int i = tid; i < H * gd; i += kPrepThreads) {          // gd decays per head: one per key channel, or one
        const float z = a[t * H * gd + i] + dt_bias[i];
        const float sp = z > 20.f ? z : log1pf(expf(z));
        gg[t * H * gd + i] = expf(-expf(a_log[i / gd]) * sp);
    }
    for (int i = tid; i < H; i += kPrepThreads) bb[t * H + i] = sigmoid_of(b[t * H + i]);
}

// One block per request; a thread owns a channel and walks its history from the oldest entry on, so that an entry is read
// before it is overwritten.
template <typename T>
__global__ void __launch_bounds__(kScanThreads)
conv_history_kernel(float* __restrict__ state, int64_t state_floats, int64_t conv_off, const T* __restrict__ packed, int stride,
                    int qkv_off, int C, int taps, const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                    int num_slots) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x;
    const int begin = cu_seqlens[s], n = cu_seqlens[s + 1] - begin;
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots || n <= 0) return;
    float* hist = state + static_cast<int64_t>(slot) * state_floats + conv_off;
    for (int c = blockIdx.y * kScanThreads + threadIdx.x; c < C; c += gridDim.y * kScanThreads) {
        for (int m = 0; m < taps - 1; ++m) {
            const int o = n - (taps - 1) + m;               // token of the portion that becomes entry m
            hist[static_cast<int64_t>(m) * C + c] = o >= 0 ? to_float(packed[static_cast<int64_t>(begin + o) * stride + qkv_off + c])
                                                           : hist[static_cast<int64_t>(n + m) * C + c];
        }
    }
}

}  // namespace cvb

using namespace cvb;

#define CVB_DISPATCH_KPT(dk, CALL)                  \
    do {                                            \
        if ((dk) <= 32) { CALL(4); }                \
        else if ((dk) <= 64) { CALL(8); }           \
        else if ((dk) <= 128) { CALL(16); }         \
        else { CALL(32); }                          \
    } while (0)

template <int KPT, int MODE>
static int launch_scan(float* out, const float* qn, const float* kn, const float* vv, const float* gg, const float* bb, const float* decay,
                       float* state, int64_t state_floats, const int* cu_seqlens, const int* state_slots, int num_slots, int S, int H, int G,
                       int dk, int dv, int* err_flag, cudaStream_t stream) {
    constexpr int arrays = MODE == 1 ? 3 : 2;
    const size_t smem = static_cast<size_t>(2) * (arrays * kScanChunk * KPT * kScanLanes + kScanChunk * kScanCols + 2 * kScanChunk) * sizeof(float);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        if (cudaFuncSetAttribute(recurrent_scan_kernel<KPT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
            return launch_status();
        raised = true;
    }
    const dim3 grid(S, H, (dv + kScanCols - 1) / kScanCols);
    launch_kernel(recurrent_scan_kernel<KPT, MODE>, grid, dim3(kScanThreads), smem, stream, out, qn, kn, vv, gg, bb, decay, state,
                  state_floats, cu_seqlens, state_slots, num_slots, H, G, dk, dv, err_flag);
    return launch_status();
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int cvb_lightning_prep(float* qf, float* kf, float* vf, const void* packed, int T, int stride, int q_off, int k_off, int v_off,
                                  int nqk, int nv, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || nqk <= 0 || nv <= 0) return CVB_E_SIZE;
    if (q_off < 0 || k_off < 0 || v_off < 0 || stride < q_off + nqk || stride < k_off + nqk || stride < v_off + nv) return CVB_E_SHAPE;
    const int64_t total = static_cast<int64_t>(T) * (2 * nqk + nv);
    const int64_t want = (total + 255) / 256;
    const unsigned blocks = static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
#define CALL(TY) launch_kernel(lightning_prep_kernel<TY>, dim3(blocks), dim3(256), 0, stream, qf, kf, vf, (const TY*)packed, stride, q_off, \
                               k_off, v_off, nqk, nv, total)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_lightning_scan(float* out, const float* qf, const float* kf, const float* vf, float* state, int64_t state_floats,
                                  const float* decay, const int* cu_seqlens, const int* state_slots, int num_slots, int S, int H, int dk,
                                  int dv, int* err_flag, cudaStream_t stream) {
    if (S == 0) return CVB_OK;
    if (S < 0 || H <= 0 || H > 65535 || dk <= 0 || dk > 256 || dv <= 0 || num_slots <= 0) return CVB_E_SIZE;
    if (state_floats < static_cast<int64_t>(H) * dk * dv) return CVB_E_SHAPE;
    if (!aligned16(qf) || !aligned16(kf) || !aligned16(vf)) return CVB_E_ALIGN;
#define CALL_K(KPT) return launch_scan<KPT, 0>(out, qf, kf, vf, nullptr, nullptr, decay, state, state_floats, cu_seqlens, state_slots, \
                                                   num_slots, S, H, H, dk, dv, err_flag, stream)
    CVB_DISPATCH_KPT(dk, CALL_K);
#undef CALL_K
}

extern "C" int cvb_delta_prep(float* qn, float* kn, float* vv, float* gg, float* bb, const void* packed, int T, int stride, int qkv_off,
                              const float* conv_w, int taps, const float* a, const float* dt_bias, const float* a_log, const float* b,
                              const float* state, int64_t state_floats, int64_t conv_off, const int* seq_of_token,
                              const int* cu_seqlens, const int* state_slots, int num_slots, int H, int G, int dk, int dv, int gd,
                              int dtype, int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || taps <= 0 || num_slots <= 0) return CVB_E_SIZE;
    const int64_t C = 2LL * G * dk + static_cast<int64_t>(H) * dv;
    if (H % G || qkv_off < 0 || stride < qkv_off + C || state_floats < conv_off + (taps - 1) * C) return CVB_E_SHAPE;
    if (gd != dk && gd != 1) return CVB_E_SHAPE;
    const size_t smem = static_cast<size_t>(2) * G * dk * sizeof(float);
    if (smem > 48 * 1024) return CVB_E_SIZE;
#define CALL(TY) launch_kernel(delta_prep_kernel<TY>, dim3(T), dim3(kPrepThreads), smem, stream, qn, kn, vv, gg, bb, (const TY*)packed, \
                               stride, qkv_off, conv_w, taps, a, dt_bias, a_log, b, state, state_floats, conv_off, seq_of_token,       \
                               cu_seqlens, state_slots, num_slots, H, G, dk, dv, gd, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_conv_history(float* state, int64_t state_floats, int64_t conv_off, const void* packed, int stride, int qkv_off, int C,
                                int taps, const int* cu_seqlens, const int* state_slots, int num_slots, int S, int dtype,
                                cudaStream_t stream) {
    if (S == 0 || taps <= 1) return CVB_OK;
    if (S < 0 || C <= 0 || num_slots <= 0) return CVB_E_SIZE;
    if (qkv_off < 0 || stride < qkv_off + C || state_floats < conv_off + static_cast<int64_t>(taps - 1) * C) return CVB_E_SHAPE;
    const dim3 grid(S, (C + kScanThreads - 1) / kScanThreads);
#define CALL(TY) launch_kernel(conv_history_kernel<TY>, grid, dim3(kScanThreads), 0, stream, state, state_floats, conv_off, \
                               (const TY*)packed, stride, qkv_off, C, taps, cu_seqlens, state_slots, num_slots)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_delta_scan(float* out, const float* qn, const float* kn, const float* vv, const float* gg, const float* bb,
                              float* state, int64_t state_floats, const int* cu_seqlens, const int* state_slots, int num_slots, int S,
                              int H, int G, int dk, int dv, int gd, int* err_flag, cudaStream_t stream) {
    if (S == 0) return CVB_OK;
    if (S < 0 || H <= 0 || H > 65535 || G <= 0 || dk <= 0 || dk > 256 || dv <= 0 || num_slots <= 0) return CVB_E_SIZE;
    if (H % G || state_floats < static_cast<int64_t>(H) * dk * dv || (gd != dk && gd != 1)) return CVB_E_SHAPE;
    if (!aligned16(qn) || !aligned16(kn) || !aligned16(vv) || !aligned16(gg)) return CVB_E_ALIGN;
    if (gd == 1 && dk != 1) {
#define CALL_K(KPT) return launch_scan<KPT, 2>(out, qn, kn, vv, gg, bb, nullptr, state, state_floats, cu_seqlens, state_slots, num_slots, \
                                               S, H, G, dk, dv, err_flag, stream)
        CVB_DISPATCH_KPT(dk, CALL_K);
#undef CALL_K
    }
#define CALL_K(KPT) return launch_scan<KPT, 1>(out, qn, kn, vv, gg, bb, nullptr, state, state_floats, cu_seqlens, state_slots, num_slots, \
                                               S, H, G, dk, dv, err_flag, stream)
    CVB_DISPATCH_KPT(dk, CALL_K);
#undef CALL_K
}
