// Grouped-query attention over cache entries that hold a key and, behind it, its value, with the masks and score terms
// that a layer switches on by its parameters:
//
//   visible keys of the token at position p:  lo <= j <= p  with
//       lo = 0                                   (all earlier tokens)
//       lo = floor(p / C) * C                    `chunk` = C > 0: only the token's own chunk, counted from position 0
//       lo = max(0, p - W + 1)                   `window` = W > 0: the last W tokens
//   and, with `pool` = P > 0 beside a window, one entry per block b of P tokens (positions bP .. bP + P - 1) that lies wholly
//   before the window, bP + P - 1 <= p - W: the means of the block's keys and values as the cache holds them, kept in a
//   second plane of the same pages at the place of position b.  Tokens and blocks share one softmax.
//   score:  s = scale * q . k;   `softcap` = c > 0:  s <- c tanh(s / c);   `r1`, `r2` [H]:  s <- s - r1_h ln(1 + r2_h (p - j))
//   (tokens only);  `sink` [H]: the softmax's denominator also holds exp(sink_h), a term without key or value;
//   `gate` [T, H]: the head's output is multiplied by sigmoid(gate[t, h]).
//
//   Pages are [plane][kv head][slot][dk + dv] with 1 plane, or 2 when blocks are pooled (plane 1: the blocks' means).
//
//   masked_qkv_prep : from the packed projection row [q: H dk | k: G dk | v: G dv]: per-head RMS norm of q and k (one weight
//                     vector for all heads, float arithmetic, one rounding), rotation of the first `rot` elements in pairs
//                     (2i, 2i + 1) or (i, i + rot / 2), the value mixed with the same token's value of an earlier layer
//                     (v <- (1 - lam) v + lam v_first), the entry's write, and the queries' write.  One warp per head.
//   pool_entries    : a step's tokens that close a block write the block's mean entry.
//   attn_masked_general : one block per (token, query head), any sizes, float or bf16: the 32-bit path and the oracle of the
//                     tensor-core forms.  Keys are walked in tiles of the block's size from the start of each run, so the
//                     order of the float sums depends only on the token's own position.
#include "common.cuh"

namespace cvb {

constexpr int kPrepWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
masked_qkv_prep_kernel(T* __restrict__ q_out, const T* __restrict__ packed, int stride, const float* __restrict__ q_w,
                       const float* __restrict__ k_w, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                       const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ pages,
                       T* __restrict__ vfirst_out, const T* __restrict__ vfirst_in, const float* __restrict__ lam_p,
                       int H, int G, int dk, int dv, int rot, int interleaved, int planes, int page_size, int max_pos, float eps,
                       int64_t total_slots, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int task = blockIdx.y * kPrepWarps + warp;
    if (task >= H + 2 * G) return;
    const int64_t t = blockIdx.x;
    const T* row = packed + t * stride;
    const int slot = slots != nullptr ? slots[t] : -1;
    const int ew = dk + dv;
    int64_t entry = -1;                                 // where this token's entry of kv head 0 starts
    if (slot >= 0 && pages != nullptr) {
        if (slot >= total_slots) {
            if (lane == 0) atomicExch(err, 2);
        } else {
            const int64_t page = slot / page_size, off = slot % page_size;
            entry = ((page * planes * G) * page_size + off) * ew;
        }
    }
    if (task >= H + G) {                                // a value head
        const int g = task - H - G;
        const T* src = row + H * dk + G * dk + g * dv;
        const float lam = (vfirst_in != nullptr && lam_p != nullptr) ? lam_p[0] : 0.f;
        for (int e = lane; e < dv; e += 32) {
            float v = to_float(src[e]);
            if (vfirst_out != nullptr) vfirst_out[t * G * dv + g * dv + e] = src[e];
            if (vfirst_in != nullptr) v = (1.f - lam) * v + lam * to_float(vfirst_in[t * G * dv + g * dv + e]);
            if (entry >= 0) pages[entry + static_cast<int64_t>(g) * page_size * ew + dk + e] = from_float<T>(v);
        }
        return;
    }
    const bool is_q = task < H;
    if (!is_q && entry < 0) return;
    const T* src = is_q ? row + task * dk : row + H * dk + (task - H) * dk;
    const float* w = is_q ? q_w : k_w;
    float* buf = smem + warp * dk;
    float ss = 0.f;
    for (int e = lane; e < dk; e += 32) { const float x = to_float(src[e]); buf[e] = x; ss = fmaf(x, x, ss); }
    if (w != nullptr) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / static_cast<float>(dk) + eps);
        for (int e = lane; e < dk; e += 32) buf[e] = buf[e] * inv * w[e];
    }
    __syncwarp();
    T* dst = is_q ? q_out + (t * H + task) * dk : pages + entry + static_cast<int64_t>(task - H) * page_size * ew;
    const int half = rot >> 1;
    if (cos_t != nullptr && half > 0) {
        int pos = positions[t];
        if (pos < 0 || pos >= max_pos) {
            if (lane == 0) atomicExch(err, 3);
            pos = pos < 0 ? 0 : max_pos - 1;
        }
        const float* c_row = cos_t + static_cast<int64_t>(pos) * half;
        const float* s_row = sin_t + static_cast<int64_t>(pos) * half;
        for (int i = lane; i < half; i += 32) {
            const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
            const float u = buf[a], v = buf[b], c = c_row[i], s = s_row[i];
            dst[a] = from_float<T>(u * c - v * s);
            dst[b] = from_float<T>(v * c + u * s);
        }
        for (int e = rot + lane; e < dk; e += 32) dst[e] = from_float<T>(buf[e]);
    } else {
        for (int e = lane; e < dk; e += 32) dst[e] = from_float<T>(buf[e]);
    }
}

// Block (token, kv head): if the token's position closes a block of `pool` positions, the mean of the block's entries (plane 0)
// goes to plane 1 at the place of position b = (p + 1) / pool - 1.  Sums run over the block's positions in rising order.
template <typename T>
__global__ void __launch_bounds__(128)
pool_entries_kernel(T* __restrict__ pages, const int* __restrict__ block_tables, int table_width, const int* __restrict__ seq_of_token,
                    const int* __restrict__ positions, int G, int ew, int pool, int page_size, int num_pages, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int g = blockIdx.y;
    const int p = positions[t];
    if (p < 0 || (p + 1) % pool != 0) return;
    const int b = (p + 1) / pool - 1;
    const int* table = block_tables + static_cast<int64_t>(seq_of_token[t]) * table_width;
    const int dst_page = b / page_size < table_width ? table[b / page_size] : -1;
    if (dst_page < 0 || dst_page >= num_pages) { if (threadIdx.x == 0) atomicExch(err, 4); return; }
    const float inv = 1.f / static_cast<float>(pool);
    for (int e = threadIdx.x; e < ew; e += blockDim.x) {
        float sum = 0.f;
        for (int j = p - pool + 1; j <= p; ++j) {
            const int page = j / page_size < table_width ? table[j / page_size] : -1;
            if (page < 0 || page >= num_pages) { atomicExch(err, 4); continue; }
            sum += to_float(pages[(((static_cast<int64_t>(page) * 2 + 0) * G + g) * page_size + j % page_size) * ew + e]);
        }
        pages[(((static_cast<int64_t>(dst_page) * 2 + 1) * G + g) * page_size + b % page_size) * ew + e] = from_float<T>(sum * inv);
    }
}

constexpr int kMaskedThreads = 128;
constexpr int kMaskedDimsPerThread = 8;

struct MaskParams {
    int chunk, window, pool;
    float scale, softcap;
};

__device__ __forceinline__ int first_visible(int p, const MaskParams& mp) {
    int lo = 0;
    if (mp.chunk > 0) lo = p / mp.chunk * mp.chunk;
    if (mp.window > 0) lo = max(lo, p - mp.window + 1);
    return lo;
}
__device__ __forceinline__ int visible_blocks(int p, const MaskParams& mp) {
    return (mp.pool > 0 && mp.window > 0) ? max(0, (p - mp.window + 1) / mp.pool) : 0;
}

template <typename T>
__global__ void __launch_bounds__(kMaskedThreads)
attn_masked_general_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ pages,
                           const int* __restrict__ block_tables, int table_width, const int* __restrict__ seq_of_token,
                           const int* __restrict__ positions, int H, int G, int dk, int dv, int page_size, int planes,
                           MaskParams mp, const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ sink,
                           const T* __restrict__ gate, int gate_stride, int num_pages, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ int64_t smem64[];
    int64_t* v_off = smem64;                            // [kMaskedThreads]
    float* probs = reinterpret_cast<float*>(v_off + kMaskedThreads);
    float* scratch = probs + kMaskedThreads;            // [32]
    float* qs = scratch + 32;                           // [dk]
    const int64_t t = blockIdx.x;
    const int h = blockIdx.y, g = h / (H / G), tid = threadIdx.x;
    const int p = positions[t];
    const int ew = dk + dv;
    const int* table = block_tables + static_cast<int64_t>(seq_of_token[t]) * table_width;
    for (int e = tid; e < dk; e += kMaskedThreads) qs[e] = to_float(q[(t * H + h) * dk + e]);
    __syncthreads();
    float acc[kMaskedDimsPerThread];
#pragma unroll
    for (int i = 0; i < kMaskedDimsPerThread; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    if (sink != nullptr) { m = sink[h]; l = 1.f; }
    const float b1 = r1 != nullptr ? r1[h] : 0.f, b2 = r2 != nullptr ? r2[h] : 0.f;
    const int lo = first_visible(p, mp), nb = visible_blocks(p, mp);
    for (int run = nb > 0 ? 0 : 1; run < 2; ++run) {
        const int first = run == 0 ? 0 : lo, last = run == 0 ? nb - 1 : p, plane = run == 0 ? 1 : 0;
        for (int start = first; start <= last; start += kMaskedThreads) {
            const int j = start + tid;
            float s = -INFINITY;
            int64_t voff = -1;
            if (j <= last) {
                const int slot = j / page_size;
                const int page = slot < table_width ? table[slot] : -1;
                if (page < 0 || page >= num_pages) {
                    atomicExch(err, 4);
                } else {
                    const int64_t koff = (((static_cast<int64_t>(page) * planes + plane) * G + g) * page_size + j % page_size) * ew;
                    voff = koff + dk;
                    const T* kp = pages + koff;
                    float d = 0.f;
                    for (int e = 0; e < dk; ++e) d = fmaf(qs[e], to_float(kp[e]), d);
                    s = d * mp.scale;
                    if (mp.softcap > 0.f) s = mp.softcap * tanhf(s / mp.softcap);
                    if (r1 != nullptr && run == 1) s -= b1 * log1pf(b2 * static_cast<float>(p - j));
                }
            }
            const float tile_max = block_max(s, scratch);
            const float m_new = fmaxf(m, tile_max);
            const float pj = (s == -INFINITY || m_new == -INFINITY) ? 0.f : expf(s - m_new);
            probs[tid] = pj;
            v_off[tid] = voff;
            const float tile_sum = block_sum(pj, scratch);
            const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
            l = l * corr + tile_sum;
            const int n = min(kMaskedThreads, last - start + 1);
#pragma unroll
            for (int i = 0; i < kMaskedDimsPerThread; ++i) {
                const int d = tid + i * kMaskedThreads;
                if (d < dv) {
                    float a = acc[i] * corr;
                    for (int jj = 0; jj < n; ++jj) {
                        const int64_t vo = v_off[jj];
                        if (vo >= 0) a = fmaf(probs[jj], to_float(pages[vo + d]), a);
                    }
                    acc[i] = a;
                }
            }
            m = m_new;
            __syncthreads();
        }
    }
    float inv_l = l > 0.f ? 1.f / l : 0.f;
    if (gate != nullptr) inv_l *= 1.f / (1.f + expf(-to_float(gate[t * gate_stride + h])));
#pragma unroll
    for (int i = 0; i < kMaskedDimsPerThread; ++i) {
        const int d = tid + i * kMaskedThreads;
        if (d < dv) out[(t * H + h) * dv + d] = from_float<T>(acc[i] * inv_l);
    }
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_masked_qkv_prep(void* q_out, const void* packed, int T, int stride, const float* q_w, const float* k_w,
                                   const float* cos_t, const float* sin_t, const int* positions, const int* slots, void* pages,
                                   void* vfirst_out, const void* vfirst_in, const float* lam, int H, int G, int dk, int dv, int rot,
                                   int interleaved, int planes, int page_size, int max_pos, float eps, int64_t total_slots, int dtype,
                                   int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || page_size <= 0) return CVB_E_SIZE;
    if (stride < H * dk + G * (dk + dv) || rot < 0 || rot > dk || (rot & 1) || (planes != 1 && planes != 2)) return CVB_E_SHAPE;
    if (rot > 0 && cos_t != nullptr && (sin_t == nullptr || positions == nullptr || max_pos <= 0)) return CVB_E_SHAPE;
    if (pages != nullptr && slots == nullptr) return CVB_E_SHAPE;
    const int tasks = H + 2 * G;
    dim3 grid(static_cast<unsigned>(T), static_cast<unsigned>((tasks + kPrepWarps - 1) / kPrepWarps));
    const size_t smem = static_cast<size_t>(kPrepWarps) * dk * sizeof(float);
    if (smem > 48 * 1024 || grid.y > 65535) return CVB_E_SIZE;
#define CALL(TY)                                                                                                          \
    launch_kernel(masked_qkv_prep_kernel<TY>, grid, dim3(kPrepWarps * 32), smem, stream, (TY*)q_out, (const TY*)packed, stride, q_w, \
                  k_w, cos_t, sin_t, positions, slots, (TY*)pages, (TY*)vfirst_out, (const TY*)vfirst_in, lam, H, G, dk, dv, rot,    \
                  interleaved, planes, page_size, max_pos, eps, total_slots, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_pool_entries(void* pages, const int* block_tables, int table_width, const int* seq_of_token, const int* positions,
                                int T, int G, int ew, int pool, int page_size, int num_pages, int dtype, int* err_flag,
                                cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || G <= 0 || ew <= 0 || pool <= 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0 || G > 65535) return CVB_E_SIZE;
#define CALL(TY)                                                                                                          \
    launch_kernel(pool_entries_kernel<TY>, dim3(T, G), dim3(128), 0, stream, (TY*)pages, block_tables, table_width, seq_of_token,   \
                  positions, G, ew, pool, page_size, num_pages, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_attn_masked_general(void* out, const void* q, const void* pages, const int* block_tables, int table_width,
                                       const int* seq_of_token, const int* positions, int T, int H, int G, int dk, int dv,
                                       int page_size, int planes, int chunk, int window, int pool, float scale, float softcap,
                                       const float* r1, const float* r2, const float* sink, const void* gate, int gate_stride,
                                       int num_pages, int dtype, int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0) return CVB_E_SIZE;
    if (dv > kMaskedThreads * kMaskedDimsPerThread || H > 65535) return CVB_E_SIZE;
    if (H % G || chunk < 0 || window < 0 || pool < 0 || (planes != 1 && planes != 2) || (pool > 0 && (planes != 2 || window <= 0)))
        return CVB_E_SHAPE;
    if ((r1 == nullptr) != (r2 == nullptr)) return CVB_E_SHAPE;
    MaskParams mp{chunk, window, pool, scale, softcap};
    const size_t smem = kMaskedThreads * sizeof(int64_t) + (static_cast<size_t>(dk) + kMaskedThreads + 32) * sizeof(float);
    if (smem > 48 * 1024) return CVB_E_SIZE;
#define CALL(TY)                                                                                                          \
    launch_kernel(attn_masked_general_kernel<TY>, dim3(T, H), dim3(kMaskedThreads), smem, stream, (TY*)out, (const TY*)q,           \
                  (const TY*)pages, block_tables, table_width, seq_of_token, positions, H, G, dk, dv, page_size, planes, mp, r1, r2, \
                  sink, (const TY*)gate, gate_stride, num_pages, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}
