// Routed feed-forward (mixture of experts): the router, the experts of a few tokens, and the experts of many.
//
//   route_topk     : z = x Wr^T + b in float (x may be bf16; Wr and b are float); top-k by z
//                    (of equal z the lower index first), weights exp(z_e) / sum over the k winners of exp(z_c):
//                    ids[t, k], weights[t, k], k in order of falling logit.  One warp per token.
//                    `mode` 1: weights scale * exp(z_e) / sum over ALL experts of exp(z_c) instead (not renormalised over the
//                    winners).  Rows of Wr behind the E experts' (`extra` of them) are not experts: their raw products
//                    leave as extra_out[t, :] (a gate per token that shares the router's pass over x).
//                    `mode` 2: weights sigmoid(z_e) of the winners, each on its own (no sum over experts at all).
//   With `on_input` = 1 a pair's weight multiplies the expert's INPUT instead of its output: y[t] = sum_k expert_e(T(w_k x[t])).
//   With `gated` = 0 an expert is  Wd_e ( T(relu(T(Wu_e x))^2) )  and Wgu holds [E, ff, D].
//   An expert is  Wd_e ( T(act(Wg_e x) * (Wu_e x)) ),  act(z) = z * sigmoid(z);  the layer's output is
//   y[t] = T( sum_k weights[t, k] * expert_{ids[t, k]}(x[t]) ).  Wgu is [E, 2 ff, D] (gate rows over up rows), Wd is
//   [E, D, ff].  Products and the weighted sum are float; the gated activation is rounded to T once, as the input of a
//   product.
//   A few tokens (decode; also the float path): two kernels that read only the chosen experts' weights, which is what
//   bounds such a step, with the work of a (token, expert) pair spread over many blocks so that every SM streams:
//     expert_hidden : block (pair, slice of ff): a warp owns inner elements, its lanes a row of the gate and of the up weight
//     expert_down   : block (token, slice of D): walks the token's experts, a warp owns output elements
//   More tokens (bf16; from a handful of tokens that share experts up to prompt portions): the (token, expert) pairs are
//   sorted by expert on the device (sort_pairs_padded: counts, every expert's segment on a multiple of 128 rows, the
//   expert of every row tile; no trip to the host, so the step stays capturable), the tokens' rows are gathered into that
//   order, two grouped products run on the tcgen05 kernel (gemm_tcgen05.cu, grouped form: gate and up rows share a tile,
//   so the gated activation is the epilogue; every chosen expert's weights are read once, experts nobody chose cost
//   nothing), and combine_pairs adds a token's expert outputs up with its weights.
#include "common.cuh"

namespace cvb {

constexpr int kRouteWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kRouteWarps * 32)
route_topk_kernel(int* __restrict__ ids, float* __restrict__ weights, const T* __restrict__ x, const float* __restrict__ wr,
                  const float* __restrict__ bias, int n_tokens, int D, int E, int top, int mode, float scale, int extra,
                  float* __restrict__ extra_out) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];                     // [kRouteWarps][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * kRouteWarps + warp;
    if (t >= n_tokens) return;
    float* z = smem + warp * E;
    const T* xr = x + t * D;
    // four rows of Wr at a time, each with a sum of its own (a row's sum runs over the same elements in the same order as
    // alone): four independent loads in flight per lane and step instead of one chain
    for (int e0 = 0; e0 < E + extra; e0 += 4) {
        const int ne = min(4, E + extra - e0);
        const float* w = wr + static_cast<int64_t>(e0) * D;
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        if (ne == 4) {
            for (int i = lane; i < D; i += 32) {
                const float xv = to_float(xr[i]);
#pragma unroll
                for (int q = 0; q < 4; ++q) d[q] = fmaf(xv, w[static_cast<int64_t>(q) * D + i], d[q]);
            }
        } else {
            for (int i = lane; i < D; i += 32) {
                const float xv = to_float(xr[i]);
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (q < ne) d[q] = fmaf(xv, w[static_cast<int64_t>(q) * D + i], d[q]);
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (q >= ne) break;
            const float v = warp_sum(d[q]);
            const int e = e0 + q;
            if (lane == 0) {
                if (e < E) z[e] = v + (bias ? bias[e] : 0.f);
                else extra_out[t * extra + (e - E)] = v;
            }
        }
    }
    __syncwarp();
    float all = 0.f;                                    // mode 1: the sum over all experts, against the largest logit
    if (mode == 1) {
        float big = -INFINITY;
        for (int e = lane; e < E; e += 32) big = fmaxf(big, z[e]);
        big = warp_max(big);
        for (int e = lane; e < E; e += 32) all += expf(z[e] - big);
        all = warp_sum(all);
    }
    float z_first = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best) { best = v; at = e; }          // the lower index wins among a lane's equals
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (k == 0) z_first = best;
        const float p = mode == 2 ? best : expf(best - z_first);      // mode 2 keeps the logit itself
        sum += p;
        if (lane == 0) {
            ids[t * top + k] = at;
            weights[t * top + k] = p;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (mode == 2) {                                    // the winners' own logistic scores
        for (int k = lane; k < top; k += 32) weights[t * top + k] = scale / (1.f + expf(-weights[t * top + k]));
        return;
    }
    const float inv = mode == 1 ? scale / all : 1.f / sum;
    for (int k = lane; k < top; k += 32) weights[t * top + k] *= inv;     // lane 0's writes are visible after the syncwarp
}

constexpr int kExpertThreads = 256;
constexpr int kExpertWarps = kExpertThreads / 32;

template <typename T> __device__ __forceinline__ float silu_exact(float g) { return g / (1.f + expf(-g)); }

// Eight weights of a bf16 row against eight floats in shared memory: one 16-byte load per lane and row.
__device__ __forceinline__ float dot8(const __nv_bfloat16* __restrict__ w, const float* __restrict__ xs, float acc) {
    const uint4 raw = *reinterpret_cast<const uint4*>(w);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float4 x0 = *reinterpret_cast<const float4*>(xs), x1 = *reinterpret_cast<const float4*>(xs + 4);
    float2 f = __bfloat1622float2(h[0]);
    acc = fmaf(x0.x, f.x, acc); acc = fmaf(x0.y, f.y, acc);
    f = __bfloat1622float2(h[1]);
    acc = fmaf(x0.z, f.x, acc); acc = fmaf(x0.w, f.y, acc);
    f = __bfloat1622float2(h[2]);
    acc = fmaf(x1.x, f.x, acc); acc = fmaf(x1.y, f.y, acc);
    f = __bfloat1622float2(h[3]);
    acc = fmaf(x1.z, f.x, acc); acc = fmaf(x1.w, f.y, acc);
    return acc;
}
template <typename T> __device__ __forceinline__ bool rows_by_16_bytes(const T*, int) { return false; }
template <> __device__ __forceinline__ bool rows_by_16_bytes<__nv_bfloat16>(const __nv_bfloat16* base, int row_len) {
    return row_len % 8 == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
}
template <typename T> __device__ __forceinline__ float dot8_of(const T*, const float*, float acc) { return acc; }
template <> __device__ __forceinline__ float dot8_of<__nv_bfloat16>(const __nv_bfloat16* w, const float* xs, float acc) { return dot8(w, xs, acc); }

// hid[pair, f] = T(silu(Wg_e[f] . x) * (Wu_e[f] . x)) for the block's slice of f; pair = t * top + k, e = ids[pair]
template <typename T>
__global__ void __launch_bounds__(kExpertThreads)
expert_hidden_kernel(T* __restrict__ hid, const T* __restrict__ x, const int* __restrict__ ids, const T* __restrict__ wgu,
                     int D, int F, int E, int top, int per_block, int gated, const float* __restrict__ in_weights,
                     int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;                                   // [D]
    const int64_t pair = blockIdx.x;
    const int64_t t = pair / top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int e = ids[pair];
    if (e < 0 || e >= E) {
        if (threadIdx.x == 0) atomicExch(err, 7);
        e = 0;
    }
    const float wi = in_weights != nullptr ? in_weights[pair] : 1.f;
    if (in_weights != nullptr) {
        for (int i = threadIdx.x; i < D; i += kExpertThreads) xs[i] = rnd<T>(wi * to_float(x[t * D + i]));
    } else {
        for (int i = threadIdx.x; i < D; i += kExpertThreads) xs[i] = to_float(x[t * D + i]);
    }
    __syncthreads();
    const T* g_rows = wgu + static_cast<int64_t>(e) * (gated ? 2 : 1) * F * D;
    const T* u_rows = g_rows + static_cast<int64_t>(F) * D;
    const int f0 = blockIdx.y * per_block, f1 = min(F, f0 + per_block);
    const bool wide = rows_by_16_bytes<T>(wgu, D);
    for (int f = f0 + warp; f < f1; f += kExpertWarps) {
        const T* gr = g_rows + static_cast<int64_t>(f) * D;
        const T* ur = u_rows + static_cast<int64_t>(f) * D;
        float g = 0.f, u = 0.f;
        if (gated) {
            for (int i = lane; i < D; i += 32) {
                const float xv = xs[i];
                g = fmaf(xv, to_float(gr[i]), g);
                u = fmaf(xv, to_float(ur[i]), u);
            }
            g = warp_sum(g);
            u = warp_sum(u);
            if (lane == 0) hid[pair * F + f] = from_float<T>(silu_exact<T>(g) * u);
        } else {
            if (wide) {
                for (int i = lane * 8; i < D; i += 256) g = dot8_of<T>(gr + i, xs + i, g);
            } else {
                for (int i = lane; i < D; i += 32) g = fmaf(xs[i], to_float(gr[i]), g);
            }
            g = fmaxf(rnd<T>(warp_sum(g)), 0.f);
            if (lane == 0) hid[pair * F + f] = from_float<T>(g * g);
        }
    }
}

// y[t, d] = T(sum_k weights[t, k] * (Wd_e[d] . hid[t * top + k])) for the block's slice of d
template <typename T>
__global__ void __launch_bounds__(kExpertThreads)
expert_down_kernel(T* __restrict__ y, const T* __restrict__ hid, const int* __restrict__ ids, const float* __restrict__ weights,
                   const T* __restrict__ wd, int D, int F, int E, int top, int per_block, int on_input) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float smem[];
    float* hs = smem;                                   // [F]
    float* acc = hs + F;                                // [per_block]
    const int64_t t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d0 = blockIdx.y * per_block, d1 = min(D, d0 + per_block);
    for (int i = threadIdx.x; i < per_block; i += kExpertThreads) acc[i] = 0.f;
    const bool wide = rows_by_16_bytes<T>(wd, F);
    for (int k = 0; k < top; ++k) {
        int e = ids[t * top + k];
        if (e < 0 || e >= E) e = 0;                      // reported by the kernel in front
        const float wk = on_input ? 1.f : weights[t * top + k];
        __syncthreads();
        for (int i = threadIdx.x; i < F; i += kExpertThreads) hs[i] = to_float(hid[(t * top + k) * F + i]);
        __syncthreads();
        const T* d_rows = wd + static_cast<int64_t>(e) * D * F;
        for (int d = d0 + warp; d < d1; d += kExpertWarps) {
            const T* dr = d_rows + static_cast<int64_t>(d) * F;
            float o = 0.f;
            if (wide) {
                for (int i = lane * 8; i < F; i += 256) o = dot8_of<T>(dr + i, hs + i, o);
            } else {
                for (int i = lane; i < F; i += 32) o = fmaf(hs[i], to_float(dr[i]), o);
            }
            o = warp_sum(o);
            if (lane == 0) acc[d - d0] = fmaf(wk, o, acc[d - d0]);     // a warp owns its d: no other warp touches acc[d - d0]
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < d1 - d0; i += kExpertThreads) y[t * D + d0 + i] = from_float<T>(acc[i]);
}

// ---- many tokens: pairs sorted by expert, grouped products on the tensor cores ------------------------------------------

constexpr int kSortThreads = 1024;

// Counts per expert, then every expert's segment of sorted rows, which starts on a multiple of `pad` rows (the tcgen05
// grouped product's row tiles are 128 rows of ONE expert).  One block.  The order of an expert's rows among themselves
// is not fixed; no result depends on it.  tile_expert[i]: the expert of row tile i, -1 for tiles behind the last segment (max_tiles
// entries).  row_token[slot]: the token whose row goes to sorted row `slot` (0 for the padding rows: they are computed
// and never read).  slot_of[pair]: where the pair's row lies.
__global__ void __launch_bounds__(kSortThreads)
sort_pairs_padded_kernel(int* __restrict__ tile_expert, int* __restrict__ row_token, int* __restrict__ slot_of,
                         const int* __restrict__ ids, int n_pairs, int E, int top, int pad, int max_tiles, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ int ismem[];
    int* count = ismem;                                 // [E]
    int* start = count + E;                             // [E + 1]
    for (int e = threadIdx.x; e < E; e += kSortThreads) count[e] = 0;
    for (int i = threadIdx.x; i < max_tiles * pad; i += kSortThreads) row_token[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += kSortThreads) {
        int e = ids[i];
        if (e < 0 || e >= E) { atomicExch(err, 7); e = 0; }
        atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) { start[e] = run; run += (count[e] + pad - 1) / pad * pad; }
        start[E] = run;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < max_tiles; i += kSortThreads) {
        int e = -1;
        if (i * pad < start[E]) {
            int lo = 0, hi = E - 1;                      // the last expert whose segment starts at or before the tile
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (start[mid] <= i * pad) lo = mid; else hi = mid - 1;
            }
            e = lo;
            while (e < E - 1 && start[e + 1] <= i * pad) ++e;      // empty experts share a start: take the one that has rows
        }
        tile_expert[i] = e;
    }
    for (int e = threadIdx.x; e < E; e += kSortThreads) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += kSortThreads) {
        int e = ids[i];
        if (e < 0 || e >= E) e = 0;
        const int slot = start[e] + atomicAdd(&count[e], 1);
        row_token[slot] = i / top;
        slot_of[i] = slot;
    }
}

// xs[slot_of[pair], :] = T(weights[pair] * x[pair / top, :]): the rows of the grouped product when a pair's weight multiplies
// the expert's input.  Padding rows keep what they held; they are computed and never read.
__global__ void scatter_pairs_scaled_kernel(__nv_bfloat16* __restrict__ xs, const __nv_bfloat16* __restrict__ x,
                                            const int* __restrict__ slot_of, const float* __restrict__ weights, int D, int top) {
    pdl_trigger();
    pdl_wait();
    const int64_t pair = blockIdx.x;
    const float w = weights[pair];
    const __nv_bfloat16* src = x + pair / top * D;
    __nv_bfloat16* dst = xs + static_cast<int64_t>(slot_of[pair]) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = __float2bfloat16_rn(w * __bfloat162float(src[d]));
}

// y[t, :] = sum_k weights[t, k] * rows[slot_of[t * top + k], :]   (weights = nullptr: all 1)
__global__ void combine_pairs_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ rows, const int* __restrict__ slot_of,
                                     const float* __restrict__ weights, int D, int top) {
    pdl_trigger();
    pdl_wait();
    const int64_t t = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k)
            s = fmaf(weights != nullptr ? weights[t * top + k] : 1.f, __bfloat162float(rows[static_cast<int64_t>(slot_of[t * top + k]) * D + d]), s);
        y[t * D + d] = __float2bfloat16_rn(s);
    }
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_route_topk(int* ids, float* weights, const void* x, const float* wr, const float* bias, int T, int D, int E,
                              int top, int mode, float scale, int extra, float* extra_out, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0 || E <= 0 || top <= 0 || extra < 0 || (extra > 0 && extra_out == nullptr)) return CVB_E_SIZE;
    if (mode < 0 || mode > 2) return CVB_E_SHAPE;
    if (top > E || E > 2048) return CVB_E_SHAPE;
    const size_t smem = static_cast<size_t>(kRouteWarps) * E * sizeof(float);
#define CALL(TY) launch_kernel(route_topk_kernel<TY>, dim3((T + kRouteWarps - 1) / kRouteWarps), dim3(kRouteWarps * 32), smem, \
                               stream, ids, weights, (const TY*)x, wr, bias, T, D, E, top, mode, scale, extra, extra_out)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_expert_rows(void* y, void* hid, const void* x, const int* ids, const float* weights, const void* wgu,
                               const void* wd, int T, int D, int F, int E, int top, int gated, int on_input, int dtype, int* err_flag,
                               cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0 || F <= 0 || E <= 0 || top <= 0) return CVB_E_SIZE;
    if (static_cast<size_t>(D) * sizeof(float) > 160 * 1024 || static_cast<size_t>(F) * sizeof(float) > 160 * 1024) return CVB_E_SIZE;
    // slices sized so that a step of one token still gives every SM a block or two
    const int64_t pairs = static_cast<int64_t>(T) * top;
    int f_per = kExpertWarps;
    while (pairs * ((F + f_per - 1) / f_per) > 1184 && f_per < F) f_per *= 2;
    int d_per = kExpertWarps;
    while (static_cast<int64_t>(T) * ((D + d_per - 1) / d_per) > 1184 && d_per < D) d_per *= 2;
    const size_t smem1 = static_cast<size_t>(D) * sizeof(float);
    const size_t smem2 = (static_cast<size_t>(F) + d_per) * sizeof(float);
    if (pairs > 2147483647LL / 2 || smem2 > 200 * 1024) return CVB_E_SIZE;
#define CALL(TY)                                                                                                         \
    do {                                                                                                                 \
        if (smem1 > 48 * 1024)                                                                                           \
            cudaFuncSetAttribute(expert_hidden_kernel<TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);     \
        if (smem2 > 48 * 1024)                                                                                           \
            cudaFuncSetAttribute(expert_down_kernel<TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);       \
        launch_kernel(expert_hidden_kernel<TY>, dim3((unsigned)pairs, (F + f_per - 1) / f_per), dim3(kExpertThreads), smem1,  \
                      stream, (TY*)hid, (const TY*)x, ids, (const TY*)wgu, D, F, E, top, f_per, gated, on_input ? weights : nullptr, err_flag);                \
        launch_kernel(expert_down_kernel<TY>, dim3(T, (D + d_per - 1) / d_per), dim3(kExpertThreads), smem2, stream,      \
                      (TY*)y, (const TY*)hid, ids, weights, (const TY*)wd, D, F, E, top, d_per, on_input);                          \
    } while (0)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

// Sorts the pairs for the tcgen05 grouped product (see sort_pairs_padded_kernel); max_tiles * 128 rows of scratch.
extern "C" int cvb_sort_pairs_padded(int* tile_expert, int* row_token, int* slot_of, const int* ids, int T, int E, int top,
                                     int max_tiles, int* err_flag, cudaStream_t stream) {
    if (T <= 0 || E <= 0 || top <= 0 || max_tiles <= 0 || E > 4096) return CVB_E_SIZE;
    const int64_t pairs = static_cast<int64_t>(T) * top;
    if (pairs > (1 << 30) || (pairs + 127) / 128 + E > max_tiles) return CVB_E_SCRATCH;
    launch_kernel(sort_pairs_padded_kernel, dim3(1), dim3(kSortThreads), (2 * static_cast<size_t>(E) + 1) * sizeof(int), stream,
                  tile_expert, row_token, slot_of, ids, static_cast<int>(pairs), E, top, 128, max_tiles, err_flag);
    return launch_status();
}

extern "C" int cvb_scatter_pairs_scaled_bf16(void* xs, const void* x, const int* slot_of, const float* weights, int T, int D, int top,
                                             cudaStream_t stream) {
    if (T <= 0 || D <= 0 || top <= 0) return CVB_E_SIZE;
    launch_kernel(scatter_pairs_scaled_kernel, dim3(static_cast<unsigned>(T) * top), dim3(D >= 1024 ? 256 : 128), 0, stream,
                  (__nv_bfloat16*)xs, (const __nv_bfloat16*)x, slot_of, weights, D, top);
    return launch_status();
}

extern "C" int cvb_combine_pairs_bf16(void* y, const void* rows, const int* slot_of, const float* weights, int T, int D, int top,
                                      cudaStream_t stream) {
    if (T <= 0 || D <= 0 || top <= 0) return CVB_E_SIZE;
    launch_kernel(combine_pairs_kernel, dim3(T), dim3(D >= 1024 ? 256 : 128), 0, stream, (__nv_bfloat16*)y,
                  (const __nv_bfloat16*)rows, slot_of, weights, D, top);
    return launch_status();
}
