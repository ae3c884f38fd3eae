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
//   attn_masked_kernel : bf16 on the tensor cores (`mma.sync.m16n8k16`, float accumulation), key and value sizes 16..128 in
//                     steps of 16.  A block owns 64 query rows of one kv head (64 / g tokens of one request times the g heads
//                     of the group) and walks 64-entry tiles gathered through the block table by 16-byte cp.async into two
//                     stages: first the pooled blocks any of its tokens sees (plane 1), then the tokens from the first one
//                     its first token sees to its last token.  One gather feeds both products (S = Q K^T from the entry's
//                     first dk columns, O += P V from the rest, read transposed).  Mask, cap, distance term and the base-2
//                     online softmax work on the score fragments in registers; a sink starts a row's maximum and sum.  Tiles
//                     are aligned to absolute positions, so a token's sums do not depend on how its prompt was cut.
#include "common.cuh"
#include "sm100.cuh"
#include "mma_tiles.cuh"

namespace cvb {

constexpr int kPrepWarps = 4;

__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ void store2(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
__device__ __forceinline__ void store2(__nv_bfloat16* p, float2 v) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y); }

constexpr int kPrepPairs = 8;                            // pairs per lane: heads of up to 512 elements

// The same epilogue two elements at a time, for even sizes and a rotation in pairs (2i, 2i + 1) (or none): a lane holds whole
// pairs in registers from the load to the store, so neither shared memory nor a second pass is needed.
template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
masked_qkv_prep_pairs_kernel(T* __restrict__ q_out, const T* __restrict__ packed, int stride, const float* __restrict__ q_w,
                             const float* __restrict__ k_w, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                             const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ pages,
                             T* __restrict__ vfirst_out, const T* __restrict__ vfirst_in, const float* __restrict__ lam_p,
                             int H, int G, int dk, int dv, int rot, int planes, int page_size, int max_pos, float eps,
                             int64_t total_slots, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int task = blockIdx.y * kPrepWarps + warp;
    if (task >= H + 2 * G) return;
    const int64_t t = blockIdx.x;
    const T* row = packed + t * stride;
    const int slot = slots != nullptr ? slots[t] : -1;
    const int ew = dk + dv;
    int64_t entry = -1;
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
        for (int e = lane * 2; e < dv; e += 64) {
            float2 v = load2(src + e);
            if (vfirst_out != nullptr) store2(vfirst_out + t * G * dv + g * dv + e, v);
            if (vfirst_in != nullptr) {
                const float2 f = load2(vfirst_in + t * G * dv + g * dv + e);
                v.x = (1.f - lam) * v.x + lam * f.x;
                v.y = (1.f - lam) * v.y + lam * f.y;
            }
            if (entry >= 0) store2(pages + entry + static_cast<int64_t>(g) * page_size * ew + dk + e, v);
        }
        return;
    }
    const bool is_q = task < H;
    if (!is_q && entry < 0) return;
    const T* src = is_q ? row + task * dk : row + H * dk + (task - H) * dk;
    const float* w = is_q ? q_w : k_w;
    const int np = dk >> 1, half = rot >> 1;
    float2 x[kPrepPairs];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kPrepPairs; ++k) {
        const int i = lane + 32 * k;
        if (i < np) { x[k] = load2(src + 2 * i); ss = fmaf(x[k].x, x[k].x, ss); ss = fmaf(x[k].y, x[k].y, ss); }
    }
    if (w != nullptr) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / static_cast<float>(dk) + eps);
#pragma unroll
        for (int k = 0; k < kPrepPairs; ++k) {
            const int i = lane + 32 * k;
            if (i < np) { x[k].x = x[k].x * inv * w[2 * i]; x[k].y = x[k].y * inv * w[2 * i + 1]; }
        }
    }
    T* dst = is_q ? q_out + (t * H + task) * dk : pages + entry + static_cast<int64_t>(task - H) * page_size * ew;
    const float* c_row = nullptr;
    const float* s_row = nullptr;
    if (cos_t != nullptr && half > 0) {
        int pos = positions[t];
        if (pos < 0 || pos >= max_pos) {
            if (lane == 0) atomicExch(err, 3);
            pos = pos < 0 ? 0 : max_pos - 1;
        }
        c_row = cos_t + static_cast<int64_t>(pos) * half;
        s_row = sin_t + static_cast<int64_t>(pos) * half;
    }
#pragma unroll
    for (int k = 0; k < kPrepPairs; ++k) {
        const int i = lane + 32 * k;
        if (i >= np) break;
        float2 v = x[k];
        if (c_row != nullptr && i < half) {
            const float c = c_row[i], s = s_row[i];
            v = make_float2(x[k].x * c - x[k].y * s, x[k].y * c + x[k].x * s);
        }
        store2(dst + 2 * i, v);
    }
}

// ---- 16 bytes per thread: head sizes whose chunk count is a power of two, a rotation in pairs (2i, 2i + 1) or none ------------
//
// One thread owns one 16-byte chunk of a head (8 bf16 or 4 float elements, whole pairs); the dk / N threads of a query or key
// head are neighbours in a warp, so the sum of squares is a butterfly over the group.  The threads of a token are laid out as
// all query and key chunks (padded to whole warps), then all value chunks.
template <typename T> struct Chunk16;
template <> struct Chunk16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(float (&v)[4], const float* p) { const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Chunk16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(float (&v)[8], const __nv_bfloat16* p) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
};

template <typename T>
__global__ void __launch_bounds__(128)
masked_qkv_prep_vec_kernel(T* __restrict__ q_out, const T* __restrict__ packed, int stride, const float* __restrict__ q_w,
                           const float* __restrict__ k_w, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                           const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ pages,
                           T* __restrict__ vfirst_out, const T* __restrict__ vfirst_in, const float* __restrict__ lam_p,
                           int H, int G, int dk, int dv, int rot, int planes, int page_size, int max_pos, float eps,
                           int64_t total_slots, int qk_pad, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    constexpr int N = Chunk16<T>::N;
    const int chk = dk / N, chv = dv / N;
    const int idx = blockIdx.y * 128 + threadIdx.x;
    const int64_t t = blockIdx.x;
    const T* row = packed + t * stride;
    const int slot = slots != nullptr ? slots[t] : -1;
    const int ew = dk + dv;
    int64_t entry = -1;
    if (slot >= 0 && pages != nullptr) {
        if (slot >= total_slots) {
            if ((threadIdx.x & 31) == 0) atomicExch(err, 2);
        } else {
            const int page = slot / page_size, off = slot - page * page_size;
            entry = ((static_cast<int64_t>(page) * planes * G) * page_size + off) * ew;
        }
    }
    float v[N];
    if (idx >= qk_pad) {                                // a chunk of a value head
        const int vi = idx - qk_pad;
        if (vi >= G * chv) return;
        const int g = vi / chv, e = (vi - g * chv) * N;
        Chunk16<T>::load(v, row + H * dk + G * dk + g * dv + e);
        if (vfirst_out != nullptr) Chunk16<T>::store(vfirst_out + t * G * dv + g * dv + e, v);
        if (vfirst_in != nullptr) {
            const float lam = lam_p[0];
            float f[N];
            Chunk16<T>::load(f, vfirst_in + t * G * dv + g * dv + e);
#pragma unroll
            for (int i = 0; i < N; ++i) v[i] = (1.f - lam) * v[i] + lam * f[i];
        }
        if (entry >= 0) Chunk16<T>::store(pages + entry + static_cast<int64_t>(g) * page_size * ew + dk + e, v);
        return;
    }
    // a chunk of a query or key head; every lane of the warp walks the butterfly, live or not
    const int task = min(idx / chk, H + G - 1), c = idx % chk;
    const bool is_q = task < H;
    const bool live = idx < (H + G) * chk && (is_q || entry >= 0);
    const float* w = is_q ? q_w : k_w;
    float ss = 0.f;
    if (live) {
        Chunk16<T>::load(v, row + task * dk + c * N);   // key heads lie behind the query heads in the row
#pragma unroll
        for (int i = 0; i < N; ++i) ss = fmaf(v[i], v[i], ss);
    }
    if (w != nullptr) {
        for (int o = chk >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = rsqrtf(ss / static_cast<float>(dk) + eps);
        if (live) {
#pragma unroll
            for (int i = 0; i < N; ++i) v[i] = v[i] * inv * w[c * N + i];
        }
    }
    if (!live) return;
    const int half = rot >> 1;
    if (cos_t != nullptr && c * N < rot) {
        int pos = positions[t];
        if (pos < 0 || pos >= max_pos) {
            atomicExch(err, 3);
            pos = pos < 0 ? 0 : max_pos - 1;
        }
        const float* c_row = cos_t + static_cast<int64_t>(pos) * half;
        const float* s_row = sin_t + static_cast<int64_t>(pos) * half;
#pragma unroll
        for (int i = 0; i < N; i += 2) {
            const int pr = (c * N + i) >> 1;
            if (pr < half) {
                const float cs = c_row[pr], sn = s_row[pr], x0 = v[i], x1 = v[i + 1];
                v[i] = x0 * cs - x1 * sn;
                v[i + 1] = x1 * cs + x0 * sn;
            }
        }
    }
    T* dst = is_q ? q_out + (t * H + task) * dk : pages + entry + static_cast<int64_t>(task - H) * page_size * ew;
    Chunk16<T>::store(dst + c * N, v);
}

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
    __shared__ int64_t off[128];                        // where the entries of up to 128 of the block's positions start
    const int64_t t = blockIdx.x;
    const int g = blockIdx.y;
    const int p = positions[t];
    if (p < 0 || (p + 1) % pool != 0) return;
    const int b = (p + 1) / pool - 1;
    const int* table = block_tables + static_cast<int64_t>(seq_of_token[t]) * table_width;
    const int dst_page = b / page_size < table_width ? table[b / page_size] : -1;
    if (dst_page < 0 || dst_page >= num_pages) { if (threadIdx.x == 0) atomicExch(err, 4); return; }
    const int64_t dst = (((static_cast<int64_t>(dst_page) * 2 + 1) * G + g) * page_size + b % page_size) * ew;
    for (int e0 = 0; e0 < ew; e0 += 512) {              // 512 elements of the entry at a time: four per thread
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j0 = p - pool + 1; j0 <= p; j0 += 128) {
            const int n = min(128, p - j0 + 1);
            __syncthreads();
            if (threadIdx.x < n) {
                const int j = j0 + threadIdx.x;
                const int page = j / page_size < table_width ? table[j / page_size] : -1;
                if (page < 0 || page >= num_pages) { atomicExch(err, 4); off[threadIdx.x] = -1; }
                else off[threadIdx.x] = (((static_cast<int64_t>(page) * 2 + 0) * G + g) * page_size + j % page_size) * ew;
            }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int e = e0 + threadIdx.x + k * 128;
                if (e >= ew) break;
                float acc = sum[k];
#pragma unroll 8
                for (int i = 0; i < n; ++i) acc += off[i] >= 0 ? to_float(pages[off[i] + e]) : 0.f;     // rising positions, one sum
                sum[k] = acc;
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int e = e0 + threadIdx.x + k * 128;
            if (e < ew) pages[dst + e] = from_float<T>(sum[k] / static_cast<float>(pool));
        }
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

// ---- bf16 on the tensor cores ------------------------------------------------------------------------------------------

constexpr int kMTileKeys = 64;
constexpr int kMTileRows = 64;
constexpr int kMThreads = 128;
constexpr float kLog2eM = 1.4426950408889634f;

struct MaskedAttnParams {
    __nv_bfloat16* out;                 // [T, H * dv]
    const __nv_bfloat16* q;             // [T, H * dk]
    const __nv_bfloat16* pages;         // [num_pages, planes, G, page_size, dk + dv]
    const __nv_bfloat16* gate;          // [T, gate_stride] or null
    const float* r1;                    // [H] or null
    const float* r2;
    const float* sink;                  // [H] or null
    const int* block_tables;            // [S, table_width]
    const int* cu_seqlens;              // [S + 1]
    const int* positions;               // [T]
    int gate_stride, table_width, S, H, G, dk, dv, page_size, page_shift, num_pages, planes;
    MaskParams mp;
    // decode form only: the tiles of a (request, kv head) are shared out among `splits` blocks (gridDim.z); with more than
    // one, a block leaves its part (unnormalised rows, maxima, sums) in `parts` and a second kernel merges them
    int splits;
    float* parts;                       // [S, G, splits, 16, dv + 2]
    int* err;
};

__device__ __forceinline__ float tanh_by_exp(float x) { return 1.f - __fdividef(2.f, 1.f + __expf(2.f * x)); }

template <int W, bool EXACT>
__global__ void __launch_bounds__(kMThreads, W <= 64 ? 3 : 2)
attn_masked_kernel(const MaskedAttnParams p) {
    pdl_trigger();
    pdl_wait();
    const int dk = EXACT ? W : p.dk, dv = EXACT ? W : p.dv;
    const int E = dk + dv;
    const int LDQ = dk + 8, LD = E + 8;                   // padded rows, in elements
    const int CQ = dk >> 3, CE = E >> 3;                  // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sK = sQ + kMTileRows * LDQ;            // two stages of kMTileKeys * LD

    const int g = p.H / p.G;
    const int tok_per_tile = kMTileRows / g;
    const int kvh = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    int seq = -1, q0 = 0, q_len = 0, cu0 = 0;
    {
        int tile = blockIdx.x;
        for (int s = 0; s < p.S; ++s) {
            const int a = p.cu_seqlens[s], n = p.cu_seqlens[s + 1] - a;
            const int tiles = (n + tok_per_tile - 1) / tok_per_tile;
            if (tile < tiles) { seq = s; q0 = tile * tok_per_tile; q_len = n; cu0 = a; break; }
            tile -= tiles;
        }
    }
    if (seq < 0) return;
    const int n_tok = min(tok_per_tile, q_len - q0);
    const int* table = p.block_tables + static_cast<int64_t>(seq) * p.table_width;
    const int pos_first = p.positions[cu0 + q0];
    const int key_hi = pos_first + n_tok - 1;             // a request's tokens of a step sit at consecutive positions
    // both bounds grow with the position: the block's first token sees the earliest token, its last one the most blocks
    const int nb_max = visible_blocks(key_hi, p.mp);
    const int n_pool_tiles = (nb_max + kMTileKeys - 1) / kMTileKeys;
    const int tok_tile0 = first_visible(pos_first, p.mp) / kMTileKeys;
    const int n_tiles = n_pool_tiles + key_hi / kMTileKeys - tok_tile0 + 1;

    for (int i = threadIdx.x; i < kMTileRows * CQ; i += kMThreads) {
        const int r = i / CQ, c = i - r * CQ;
        const int tok = r / g;
        const bool valid = tok < n_tok;
        const __nv_bfloat16* src = valid ? p.q + (static_cast<int64_t>(cu0 + q0 + tok) * p.H + kvh * g + r % g) * dk + c * 8 : p.q;
        cp_async16(sQ + r * LDQ + c * 8, src, valid);
    }

    const int ld_r0 = threadIdx.x / CE, ld_c0 = threadIdx.x - ld_r0 * CE;
    const int ld_dr = kMThreads / CE, ld_dc = kMThreads - ld_dr * CE;
    auto load_tile = [&](int it, int stage) {
        const bool pooled = it < n_pool_tiles;
        const int key0 = pooled ? it * kMTileKeys : (tok_tile0 + it - n_pool_tiles) * kMTileKeys;
        const int hi = pooled ? nb_max - 1 : key_hi;
        const int plane = pooled ? 1 : 0;
        __nv_bfloat16* dst = sK + stage * kMTileKeys * LD;
        int last_slot = -1, page = -1;                    // a thread's rows ascend: the block table is read once per page
        int r = ld_r0, c = ld_c0;
        for (; r < kMTileKeys; r += ld_dr, c += ld_dc) {
            if (c >= CE) { c -= CE; ++r; if (r >= kMTileKeys) break; }
            const int j = key0 + r;
            bool need = j <= hi;
            const __nv_bfloat16* src = p.pages;
            if (need) {
                int slot, off;
                if (p.page_shift >= 0) { slot = j >> p.page_shift; off = j & (p.page_size - 1); }
                else { slot = j / p.page_size; off = j - slot * p.page_size; }
                if (slot != last_slot) { page = slot < p.table_width ? table[slot] : -1; last_slot = slot; }
                if (page < 0 || page >= p.num_pages) {
                    atomicExch(p.err, 4);                 // an entry a token of this block must see has no page
                    need = false;
                } else {
                    src = p.pages + (((static_cast<int64_t>(page) * p.planes + plane) * p.G + kvh) * p.page_size + off) * E + c * 8;
                }
            }
            cp_async16(dst + r * LD + c * 8, src, need);
        }
    };

    load_tile(0, 0);
    cp_async_commit();

    // the two rows this thread owns in its warp's slab of 16
    int ptok[2], lo_t[2], nb_t[2];
    float b1[2] = {0.f, 0.f}, b2[2] = {0.f, 0.f};
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + (lane >> 2) + half * 8;
        const int tok = min(r / g, n_tok - 1);            // rows past the block's tokens are never stored
        const int head = kvh * g + r % g;
        ptok[half] = pos_first + tok;
        lo_t[half] = first_visible(ptok[half], p.mp);
        nb_t[half] = visible_blocks(ptok[half], p.mp);
        if (p.r1 != nullptr) { b1[half] = p.r1[head]; b2[half] = p.r2[head]; }
        if (p.sink != nullptr) { m[half] = p.sink[head] * kLog2eM; l[half] = (lane & 3) == 0 ? 1.f : 0.f; }
    }
    const bool warp_has_rows = warp * 16 < n_tok * g;
    const int warp_first_pos = pos_first + min(n_tok - 1, (warp * 16) / g);
    const int warp_last_pos = pos_first + min(n_tok - 1, (warp * 16 + 15) / g);
    const int warp_lo = first_visible(warp_first_pos, p.mp), warp_nb = visible_blocks(warp_last_pos, p.mp);
    const float cap = p.mp.softcap, inv_cap = cap > 0.f ? 1.f / cap : 0.f;

    float o[W / 8][4];
#pragma unroll
    for (int dt = 0; dt < W / 8; ++dt) { o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f; }
    uint32_t qf[W / 16][4];

    for (int it = 0; it < n_tiles; ++it) {
        if (it + 1 < n_tiles) load_tile(it + 1, (it + 1) & 1);
        cp_async_commit();
        const bool pooled = it < n_pool_tiles;
        const int key0 = pooled ? it * kMTileKeys : (tok_tile0 + it - n_pool_tiles) * kMTileKeys;
        cp_async_wait<1>();                               // everything but the newest group: the query tile and tile `it`
        __syncthreads();
        if (it == 0) {
#pragma unroll
            for (int ks = 0; ks < W / 16; ++ks) {
                if (!EXACT && ks * 16 >= dk) break;
                ldm_x4(qf[ks], sQ + (warp * 16 + (lane & 15)) * LDQ + ks * 16 + (lane >> 4) * 8);
            }
        }
        const bool wanted = pooled ? key0 < warp_nb : (key0 <= warp_last_pos && key0 + kMTileKeys - 1 >= warp_lo);
        if (warp_has_rows && wanted) {
            const __nv_bfloat16* tile = sK + (it & 1) * kMTileKeys * LD;
            float s[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < W / 16; ++ks) {
                if (!EXACT && ks * 16 >= dk) break;
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b[4];
                    ldm_x4(b, tile + (np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
                    mma_16816(s[np * 2], qf[ks], b[0], b[1]);
                    mma_16816(s[np * 2 + 1], qf[ks], b[2], b[3]);
                }
            }
            // scale, cap, distance term, mask; running maximum
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int half = e >> 1;
                    const int j = key0 + nt * 8 + ((lane & 3) << 1) + (e & 1);
                    const bool visible = pooled ? j < nb_t[half] : (j >= lo_t[half] && j <= ptok[half]);
                    float v = s[nt][e] * p.mp.scale;
                    if (cap > 0.f) v = cap * tanh_by_exp(v * inv_cap);
                    if (p.r1 != nullptr && !pooled) v -= b1[half] * __logf(1.f + b2[half] * static_cast<float>(max(ptok[half] - j, 0)));
                    v = visible ? v * kLog2eM : -INFINITY;
                    s[nt][e] = v;
                    mx[half] = fmaxf(mx[half], v);
                }
            }
            float corr[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 1));
                mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 2));
                const float m_new = fmaxf(m[half], mx[half]);
                corr[half] = (m[half] == -INFINITY) ? 0.f : ex2(m[half] - m_new);
                m[half] = m_new;
            }
            float sum[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int half = e >> 1;
                    const float pj = (s[nt][e] == -INFINITY) ? 0.f : ex2(s[nt][e] - m[half]);
                    s[nt][e] = pj;
                    sum[half] += pj;
                }
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) l[half] = l[half] * corr[half] + sum[half];
#pragma unroll
            for (int dt = 0; dt < W / 8; ++dt) {
                o[dt][0] *= corr[0]; o[dt][1] *= corr[0]; o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
            }
            // O += P V: the columns behind the keys, read transposed
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t a[4];
                a[0] = pack2(s[kk * 2][0], s[kk * 2][1]);
                a[1] = pack2(s[kk * 2][2], s[kk * 2][3]);
                a[2] = pack2(s[kk * 2 + 1][0], s[kk * 2 + 1][1]);
                a[3] = pack2(s[kk * 2 + 1][2], s[kk * 2 + 1][3]);
#pragma unroll
                for (int dp = 0; dp < W / 16; ++dp) {
                    if (!EXACT && dp * 16 >= dv) break;
                    uint32_t b[4];
                    ldm_x4_trans(b, tile + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dk + dp * 16 + ((lane >> 4) & 1) * 8);
                    mma_16816(o[dp * 2], a, b[0], b[1]);
                    mma_16816(o[dp * 2 + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                  // the stage may be filled again
    }

#pragma unroll
    for (int half = 0; half < 2; ++half) {
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 1);
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 2);
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + (lane >> 2) + half * 8;
        const int tok = r / g;
        if (tok >= n_tok) continue;
        const int head = kvh * g + r % g;
        float inv = l[half] > 0.f ? 1.f / l[half] : 0.f;
        if (p.gate != nullptr)
            inv *= 1.f / (1.f + __expf(-__bfloat162float(p.gate[static_cast<int64_t>(cu0 + q0 + tok) * p.gate_stride + head])));
        __nv_bfloat16* dst = p.out + (static_cast<int64_t>(cu0 + q0 + tok) * p.H + head) * dv;
#pragma unroll
        for (int dt = 0; dt < W / 8; ++dt) {
            const int d = dt * 8 + ((lane & 3) << 1);
            if (!EXACT && d >= dv) break;
            *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(o[dt][half * 2] * inv, o[dt][half * 2 + 1] * inv);
        }
    }
}

template <int W, bool EXACT>
int launch_attn_masked(const MaskedAttnParams& p, int num_tiles, cudaStream_t stream) {
    const int E = p.dk + p.dv;
    const size_t smem = (static_cast<size_t>(kMTileRows) * (p.dk + 8) + static_cast<size_t>(2) * kMTileKeys * (E + 8)) * sizeof(__nv_bfloat16);
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(attn_masked_kernel<W, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)
            return launch_status();
        raised = true;
    }
    launch_kernel(attn_masked_kernel<W, EXACT>, dim3(num_tiles, p.G), dim3(kMThreads), smem, stream, p);
    return launch_status();
}

// ---- decoded tokens: one token per request ---------------------------------------------------------------------------
//
// A block owns one (request, kv head): the g <= 16 query heads of the group are the rows of ONE 16-row slab, and each of
// the block's warps takes every n-th tile of 32 entries (first the pooled blocks the token sees, then its tokens from the
// first visible one) into two stages of its own: cp.async by its own lanes, __syncwarp, no block-wide barrier in the loop.
// The warps' parts are merged through shared memory; when few (request, kv head) pairs would leave SMs idle the tiles are
// shared out among `splits` blocks as well, which leave their parts in scratch for a merge kernel.  The sink and the gate
// join where the parts are merged, once.
constexpr int kMDecKeys = 32;

__device__ __forceinline__ void masked_finish(const MaskedAttnParams& p, int t, int head, int d, int dv, float mm, float ll, float acc) {
    if (p.sink != nullptr) {
        const float sk = p.sink[head] * kLog2eM;
        const float top = fmaxf(mm, sk);
        const float f = mm == -INFINITY ? 0.f : ex2(mm - top);
        ll = ll * f + ex2(sk - top);
        acc *= f;
    }
    float v = ll > 0.f ? acc / ll : 0.f;
    if (p.gate != nullptr) v *= 1.f / (1.f + __expf(-__bfloat162float(p.gate[static_cast<int64_t>(t) * p.gate_stride + head])));
    p.out[(static_cast<int64_t>(t) * p.H + head) * dv + d] = __float2bfloat16_rn(v);
}

template <int W, bool EXACT>
__global__ void __launch_bounds__(256)
attn_masked_decode_kernel(const MaskedAttnParams p) {
    pdl_trigger();
    pdl_wait();
    const int dk = EXACT ? W : p.dk, dv = EXACT ? W : p.dv;
    const int E = dk + dv;
    const int LDQ = dk + 8, LD = E + 8;
    const int CQ = dk >> 3, CE = E >> 3;
    const int nw = blockDim.x >> 5;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);                    // [16][LDQ]
    __nv_bfloat16* sK = sQ + 16 * LDQ;                                                 // [warps][2][32][LD]
    float* red_ml = reinterpret_cast<float*>(sK + nw * 2 * kMDecKeys * LD);            // [warps][16][2]
    const int g = p.H / p.G;
    const int seq = blockIdx.x, kvh = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = p.cu_seqlens[seq];
    const int pos = p.positions[t];
    const int* table = p.block_tables + static_cast<int64_t>(seq) * p.table_width;
    const int lo = first_visible(pos, p.mp), nb = visible_blocks(pos, p.mp);
    const int n_pool_tiles = (nb + kMDecKeys - 1) / kMDecKeys;
    const int tok_tile0 = lo / kMDecKeys;
    const int n_tiles = n_pool_tiles + pos / kMDecKeys - tok_tile0 + 1;

    for (int i = threadIdx.x; i < 16 * CQ; i += blockDim.x) {
        const int r = i / CQ, c = i - r * CQ;
        const bool valid = r < g;
        cp_async16(sQ + r * LDQ + c * 8, valid ? p.q + (static_cast<int64_t>(t) * p.H + kvh * g + r) * dk + c * 8 : p.q, valid);
    }
    cp_async_commit();

    __nv_bfloat16* my = sK + warp * 2 * kMDecKeys * LD;
    const int ld_r0 = lane / CE, ld_c0 = lane - ld_r0 * CE;
    const int ld_dr = 32 / CE, ld_dc = 32 - ld_dr * CE;
    auto load_tile = [&](int it, int stage) {
        const bool pooled = it < n_pool_tiles;
        const int key0 = pooled ? it * kMDecKeys : (tok_tile0 + it - n_pool_tiles) * kMDecKeys;
        const int hi = pooled ? nb - 1 : pos;
        const int plane = pooled ? 1 : 0;
        __nv_bfloat16* dst = my + stage * kMDecKeys * LD;
        int last_slot = -1, page = -1;
        const __nv_bfloat16* page_base = p.pages;
        int r = ld_r0, c = ld_c0;                         // chunk lane + 32 n is row (lane + 32 n) / CE: kept by increments
        if (p.page_shift >= 5) {
            // pages of 32 tokens and more (a power of two): the tile lies in ONE page, its rows side by side
            const int slot = key0 >> p.page_shift;
            page = slot < p.table_width ? table[slot] : -1;
            const bool ok = page >= 0 && page < p.num_pages;
            if (!ok) atomicExch(p.err, 4);
            const __nv_bfloat16* base = ok ? p.pages + (((static_cast<int64_t>(page) * p.planes + plane) * p.G + kvh) * p.page_size
                                                        + (key0 & (p.page_size - 1))) * E : p.pages;
            const int live = ok ? hi - key0 : -1;         // rows 0..live hold entries the token may see
            for (; r < kMDecKeys; r += ld_dr, c += ld_dc) {
                if (c >= CE) { c -= CE; ++r; if (r >= kMDecKeys) break; }
                const bool need = r <= live;
                cp_async16(dst + r * LD + c * 8, need ? base + r * E + c * 8 : p.pages, need);
            }
            return;
        }
        for (; r < kMDecKeys; r += ld_dr, c += ld_dc) {
            if (c >= CE) { c -= CE; ++r; if (r >= kMDecKeys) break; }
            const int j = key0 + r;
            bool need = j <= hi;
            const __nv_bfloat16* src = p.pages;
            if (need) {
                int slot, off;
                if (p.page_shift >= 0) { slot = j >> p.page_shift; off = j & (p.page_size - 1); }
                else { slot = j / p.page_size; off = j - slot * p.page_size; }
                if (slot != last_slot) {
                    page = slot < p.table_width ? table[slot] : -1;
                    last_slot = slot;
                    page_base = p.pages + ((static_cast<int64_t>(page) * p.planes + plane) * p.G + kvh) * p.page_size * E;
                }
                if (page < 0 || page >= p.num_pages) {
                    atomicExch(p.err, 4);
                    need = false;
                } else {
                    src = page_base + off * E + c * 8;
                }
            }
            cp_async16(dst + r * LD + c * 8, src, need);
        }
    };

    const int lanes_w = nw * p.splits;                    // warps that share the tiles: this block's and its siblings'
    const int gw = blockIdx.z * nw + warp;
    const int my_tiles = n_tiles > gw ? (n_tiles - gw + lanes_w - 1) / lanes_w : 0;     // tiles gw, gw + lanes_w, ...
    if (my_tiles > 0) load_tile(gw, 0);
    cp_async_commit();
    cp_async_wait<1>();                                   // this thread's share of the queries
    __syncthreads();                                      // everybody's share
    uint32_t qf[W / 16][4];
#pragma unroll
    for (int ks = 0; ks < W / 16; ++ks) {
        if (!EXACT && ks * 16 >= dk) break;
        ldm_x4(qf[ks], sQ + (lane & 15) * LDQ + ks * 16 + (lane >> 4) * 8);
    }
    float b1[2] = {0.f, 0.f}, b2[2] = {0.f, 0.f};
    if (p.r1 != nullptr) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = min((lane >> 2) + half * 8, g - 1);   // rows past the group repeat its last head; never stored
            b1[half] = p.r1[kvh * g + r];
            b2[half] = p.r2[kvh * g + r];
        }
    }
    const float cap = p.mp.softcap, inv_cap = cap > 0.f ? 1.f / cap : 0.f;

    float o[W / 8][4];
#pragma unroll
    for (int dt = 0; dt < W / 8; ++dt) { o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int n = 0; n < my_tiles; ++n) {
        const int it = gw + n * lanes_w;
        if (n + 1 < my_tiles) load_tile(it + lanes_w, (n + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();
        const bool pooled = it < n_pool_tiles;
        const int key0 = pooled ? it * kMDecKeys : (tok_tile0 + it - n_pool_tiles) * kMDecKeys;
        const __nv_bfloat16* tile = my + (n & 1) * kMDecKeys * LD;
        float s[kMDecKeys / 8][4];
#pragma unroll
        for (int nt = 0; nt < kMDecKeys / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < W / 16; ++ks) {
            if (!EXACT && ks * 16 >= dk) break;
#pragma unroll
            for (int np = 0; np < kMDecKeys / 16; ++np) {
                uint32_t b[4];
                ldm_x4(b, tile + (np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_16816(s[np * 2], qf[ks], b[0], b[1]);
                mma_16816(s[np * 2 + 1], qf[ks], b[2], b[3]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < kMDecKeys / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int half = e >> 1;
                const int j = key0 + nt * 8 + ((lane & 3) << 1) + (e & 1);
                const bool visible = pooled ? j < nb : (j >= lo && j <= pos);
                float v = s[nt][e] * p.mp.scale;
                if (cap > 0.f) v = cap * tanh_by_exp(v * inv_cap);
                if (p.r1 != nullptr && !pooled) v -= b1[half] * __logf(1.f + b2[half] * static_cast<float>(max(pos - j, 0)));
                v = visible ? v * kLog2eM : -INFINITY;
                s[nt][e] = v;
                mx[half] = fmaxf(mx[half], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 1));
            mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 2));
            const float m_new = fmaxf(m[half], mx[half]);
            corr[half] = (m[half] == -INFINITY) ? 0.f : ex2(m[half] - m_new);
            m[half] = m_new;
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < kMDecKeys / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pj = (s[nt][e] == -INFINITY) ? 0.f : ex2(s[nt][e] - m[e >> 1]);
                s[nt][e] = pj;
                sum[e >> 1] += pj;
            }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) l[half] = l[half] * corr[half] + sum[half];
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {     // no row's maximum moved: nothing to rescale
#pragma unroll
            for (int dt = 0; dt < W / 8; ++dt) {
                o[dt][0] *= corr[0]; o[dt][1] *= corr[0]; o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
            }
        }
#pragma unroll
        for (int kk = 0; kk < kMDecKeys / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack2(s[kk * 2][0], s[kk * 2][1]);
            a[1] = pack2(s[kk * 2][2], s[kk * 2][3]);
            a[2] = pack2(s[kk * 2 + 1][0], s[kk * 2 + 1][1]);
            a[3] = pack2(s[kk * 2 + 1][2], s[kk * 2 + 1][3]);
#pragma unroll
            for (int dp = 0; dp < W / 16; ++dp) {
                if (!EXACT && dp * 16 >= dv) break;
                uint32_t b[4];
                ldm_x4_trans(b, tile + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dk + dp * 16 + ((lane >> 4) & 1) * 8);
                mma_16816(o[dp * 2], a, b[0], b[1]);
                mma_16816(o[dp * 2 + 1], a, b[2], b[3]);
            }
        }
        __syncwarp();                                     // the stage may be filled again
    }
    cp_async_wait<0>();

    // merge the warps' parts: each leaves its sums, maxima and its accumulator [16][dv] (float) in its own stages
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 1);
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 2);
    }
    __syncwarp();
    float* part = reinterpret_cast<float*>(my);            // 16 * dv floats = 64 * dv bytes, within the warp's two stages (128 * LD bytes)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = (lane >> 2) + half * 8;
        if ((lane & 3) == 0) { red_ml[(warp * 16 + r) * 2] = m[half]; red_ml[(warp * 16 + r) * 2 + 1] = l[half]; }
#pragma unroll
        for (int dt = 0; dt < W / 8; ++dt) {
            const int d = dt * 8 + ((lane & 3) << 1);
            if (!EXACT && d >= dv) break;
            part[r * dv + d] = o[dt][half * 2];
            part[r * dv + d + 1] = o[dt][half * 2 + 1];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < g * dv; i += blockDim.x) {
        const int r = i / dv, d = i - r * dv;
        float mm = -INFINITY;
        for (int w = 0; w < nw; ++w) mm = fmaxf(mm, red_ml[(w * 16 + r) * 2]);
        float ll = 0.f, acc = 0.f;
        for (int w = 0; w < nw; ++w) {
            const float mw = red_ml[(w * 16 + r) * 2];
            const float f = mw == -INFINITY ? 0.f : ex2(mw - mm);
            ll += red_ml[(w * 16 + r) * 2 + 1] * f;
            acc += reinterpret_cast<const float*>(sK + w * 2 * kMDecKeys * LD)[r * dv + d] * f;
        }
        if (p.splits == 1) {
            masked_finish(p, t, kvh * g + r, d, dv, mm, ll, acc);
        } else {
            float* dst = p.parts + ((static_cast<int64_t>(seq) * p.G + kvh) * p.splits + blockIdx.z) * 16 * (dv + 2) + r * (dv + 2);
            dst[d] = acc;
            if (d == 0) { dst[dv] = mm; dst[dv + 1] = ll; }
        }
    }
}

// out = the parts of a (request, kv head) added up: rows scaled to the common maximum, divided by the common sum
__global__ void attn_masked_merge_kernel(const MaskedAttnParams p) {
    pdl_trigger();
    pdl_wait();
    const int g = p.H / p.G, dv = p.dv;
    const int seq = blockIdx.x, kvh = blockIdx.y;
    const int t = p.cu_seqlens[seq];
    const float* base = p.parts + (static_cast<int64_t>(seq) * p.G + kvh) * p.splits * 16 * (dv + 2);
    for (int i = blockIdx.z * blockDim.x + threadIdx.x; i < g * dv; i += gridDim.z * blockDim.x) {
        const int r = i / dv, d = i - r * dv;
        float mm = -INFINITY;
        for (int z = 0; z < p.splits; ++z) mm = fmaxf(mm, base[(z * 16 + r) * (dv + 2) + dv]);
        float ll = 0.f, acc = 0.f;
        for (int z = 0; z < p.splits; ++z) {
            const float* row = base + (z * 16 + r) * (dv + 2);
            const float f = row[dv] == -INFINITY ? 0.f : ex2(row[dv] - mm);
            ll += row[dv + 1] * f;
            acc += row[d] * f;
        }
        masked_finish(p, t, kvh * g + r, d, dv, mm, ll, acc);
    }
}

template <int W, bool EXACT>
int launch_attn_masked_decode(const MaskedAttnParams& p, cudaStream_t stream) {
    const int E = p.dk + p.dv;
    // as many warps as their stages leave room for, eight at most
    const size_t per_warp = static_cast<size_t>(2) * kMDecKeys * (E + 8) * sizeof(__nv_bfloat16) + 16 * 2 * sizeof(float);
    const size_t room = 216 * 1024 - static_cast<size_t>(16) * (p.dk + 8) * sizeof(__nv_bfloat16);
    const int nw = room / per_warp >= 8 ? 8 : static_cast<int>(room / per_warp);
    const size_t smem = (static_cast<size_t>(16) * (p.dk + 8) + static_cast<size_t>(nw) * 2 * kMDecKeys * (E + 8)) * sizeof(__nv_bfloat16)
                        + nw * 16 * 2 * sizeof(float);
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(attn_masked_decode_kernel<W, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024) != cudaSuccess)
            return launch_status();
        raised = true;
    }
    launch_kernel(attn_masked_decode_kernel<W, EXACT>, dim3(p.S, p.G, p.splits), dim3(nw * 32), smem, stream, p);
    if (p.splits > 1) launch_kernel(attn_masked_merge_kernel, dim3(p.S, p.G, (p.H / p.G * p.dv + 127) / 128), dim3(128), 0, stream, p);
    return launch_status();
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
    const bool turns = rot > 0 && cos_t != nullptr;
    const bool pairs = dk % 2 == 0 && dv % 2 == 0 && stride % 2 == 0 && dk <= 64 * kPrepPairs && (interleaved || !turns)
                       && ((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(pages)
                            | reinterpret_cast<uintptr_t>(vfirst_out) | reinterpret_cast<uintptr_t>(vfirst_in)) & 7) == 0;
    // 16 bytes per thread where a head is a power of two of such chunks and everything is aligned to them
    const int n16 = dtype == CVB_DTYPE_BF16 ? 8 : 4;
    const int chk = dk / n16;
    const bool vec16 = pairs && dk % n16 == 0 && dv % n16 == 0 && stride % n16 == 0 && chk <= 32 && (chk & (chk - 1)) == 0 && rot % 2 == 0
                       && ((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(pages)
                            | reinterpret_cast<uintptr_t>(vfirst_out) | reinterpret_cast<uintptr_t>(vfirst_in)) & 15) == 0;
    const int qk_pad = vec16 ? ((H + G) * chk + 31) / 32 * 32 : 0;
    const dim3 grid16(static_cast<unsigned>(T), vec16 ? static_cast<unsigned>((qk_pad + G * (dv / n16) + 127) / 128) : 1u);
#define CALL(TY)                                                                                                          \
    if (vec16)                                                                                                            \
    launch_kernel(masked_qkv_prep_vec_kernel<TY>, grid16, dim3(128), 0, stream, (TY*)q_out, (const TY*)packed, stride, q_w,           \
                  k_w, cos_t, sin_t, positions, slots, (TY*)pages, (TY*)vfirst_out, (const TY*)vfirst_in, lam, H, G, dk, dv, rot,    \
                  planes, page_size, max_pos, eps, total_slots, qk_pad, err_flag);                                        \
    else if (pairs)                                                                                                       \
    launch_kernel(masked_qkv_prep_pairs_kernel<TY>, grid, dim3(kPrepWarps * 32), 0, stream, (TY*)q_out, (const TY*)packed, stride, q_w, \
                  k_w, cos_t, sin_t, positions, slots, (TY*)pages, (TY*)vfirst_out, (const TY*)vfirst_in, lam, H, G, dk, dv, rot,    \
                  planes, page_size, max_pos, eps, total_slots, err_flag);                                                \
    else                                                                                                                  \
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

// 1 if the tensor-core kernel takes this shape: bf16, key and value sizes 16..128 in steps of 16, up to 64 query heads per kv head.
extern "C" int cvb_attn_masked_supported(int H, int G, int dk, int dv) {
    return (H > 0 && G > 0 && H % G == 0 && H / G <= kMTileRows && dk >= 16 && dk <= 128 && dk % 16 == 0
            && dv >= 16 && dv <= 128 && dv % 16 == 0) ? 1 : 0;
}

extern "C" int cvb_attn_masked_bf16(void* out, const void* q, const void* pages, const int* block_tables, int table_width,
                                    const int* cu_seqlens, const int* positions, int S, int num_tiles, int H, int G, int dk, int dv,
                                    int page_size, int planes, int chunk, int window, int pool, float scale, float softcap,
                                    const float* r1, const float* r2, const float* sink, const void* gate, int gate_stride,
                                    int num_pages, int all_single, int splits, float* parts, int64_t parts_floats, int* err_flag,
                                    cudaStream_t stream) {
    if (num_tiles == 0 || S == 0) return CVB_OK;
    if (S < 0 || num_tiles < 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0) return CVB_E_SIZE;
    if (!cvb_attn_masked_supported(H, G, dk, dv)) return CVB_E_UNSUPPORTED;
    if (chunk < 0 || window < 0 || pool < 0 || (planes != 1 && planes != 2) || (pool > 0 && (planes != 2 || window <= 0))) return CVB_E_SHAPE;
    if ((r1 == nullptr) != (r2 == nullptr)) return CVB_E_SHAPE;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(pages) | reinterpret_cast<uintptr_t>(out)) & 15) return CVB_E_ALIGN;
    if (G > 65535) return CVB_E_SIZE;
    MaskedAttnParams p;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.pages = static_cast<const __nv_bfloat16*>(pages);
    p.gate = static_cast<const __nv_bfloat16*>(gate); p.gate_stride = gate_stride;
    p.r1 = r1; p.r2 = r2; p.sink = sink;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.table_width = table_width; p.S = S; p.H = H; p.G = G; p.dk = dk; p.dv = dv; p.page_size = page_size;
    p.num_pages = num_pages; p.planes = planes;
    p.page_shift = -1;
    for (int sh = 0; sh < 31; ++sh)
        if ((1 << sh) == page_size) p.page_shift = sh;
    p.mp = MaskParams{chunk, window, pool, scale, softcap};
    p.err = err_flag;
    p.splits = 1; p.parts = nullptr;
    const bool decode = all_single && H / G <= 16;        // every request brings one token: the kernel for decoded tokens
    if (decode && splits > 1) {
        if (splits > 64) return CVB_E_SIZE;
        if (parts == nullptr || parts_floats < static_cast<int64_t>(S) * G * splits * 16 * (dv + 2)) return CVB_E_SCRATCH;
        p.splits = splits; p.parts = parts;
    }
    const int w = dk > dv ? dk : dv;
    const bool exact = dk == dv && (dk == 64 || dk == 128);
#define CVB_MASKED_WIDTH(WW)                                                                                             \
    if (w <= WW) {                                                                                                       \
        if (decode) return exact ? launch_attn_masked_decode<WW, true>(p, stream) : launch_attn_masked_decode<WW, false>(p, stream); \
        return exact ? launch_attn_masked<WW, true>(p, num_tiles, stream) : launch_attn_masked<WW, false>(p, num_tiles, stream);     \
    }
    CVB_MASKED_WIDTH(64)
    CVB_MASKED_WIDTH(128)
#undef CVB_MASKED_WIDTH
    return CVB_E_UNSUPPORTED;
}
