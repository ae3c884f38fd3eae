// General paged attention: any head size, any number of heads and groups, float or bf16, optional window, optional kept
// first positions, pages that hold keys and values or keys that are also the values.
// One block per (query token, query head).  It serves prompt portions and decoded tokens alike, because
// every query token is handled on its own: its keys are those of its request at positions lo..p, read
// through the request's block table, where p is the token's absolute position and lo = 0 or, with a
// window w > 0, max(0, p - w + 1).  With `keep_first` = f > 0 the positions 0..f-1 stay visible after the window has
// passed them: the token then reads 0..min(f, lo)-1 and lo..p (two runs of tiles).  The keys of the step's own tokens
// are already in the pages (the projection kernel writes before this kernel reads).  `planes` = 2: a page is
// [K | V][kv head][slot][hd]; `planes` = 1: a page is [kv head][slot][hd] and a key is also its value.  Queries are
// read from rows of `q_stride` elements (the packed output of a projection, or [T, H, hd] itself).  With `planes` = 1 the
// value may be narrower than the key: `vd` <= hd says how many leading elements of a key are its value (a cache of latent
// vectors with a positional part behind them); the output rows are [T, H, vd].  More generally with `planes` = 1 an entry
// of a kv head is `ew` >= hd elements wide, its first hd elements are the key and the vd elements from `voff` on are the
// value (ew = hd, voff = 0: the key's leading elements; ew = hd + vd, voff = hd: a key with its own value behind it, of
// any size).  With a distance table `bias` [H, bias_len] (float) the score receives bias[h, min(p - j, bias_len - 1)] after
// the scale: a learned bias per head and distance, whose last entry serves every larger distance.
//
// Formulas (reference kernels/paged_attention.cu:89-359 and model/model_architecture.cpp:134,147):
//   query head h uses kv head h / (H / KV);  s_j = scale * q . k_j  for lo <= j <= p, others excluded;
//   running maximum m, sum l and accumulator in float with expf;  o = sum_j p_j v_j / l;  rounded to T.
// Keys are walked in tiles of blockDim.x from the start of each run, so the order of the float sums depends only on (f, lo, p):
// not on how the prompt was cut into steps, nor on the batch, nor on which pages hold the keys.
#include "common.cuh"

namespace cvb {

constexpr int kAttnThreads = 128;
constexpr int kMaxDimsPerThread = 8;     // head sizes up to 1024

template <typename T>
__global__ void __launch_bounds__(kAttnThreads)
paged_attention_general_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ cache,
                               const int* __restrict__ block_tables, int table_width,
                               const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                               int H, int KV, int hd, int vd, int page_size, int window, int keep_first, int planes, int q_stride,
                               float scale, int num_pages, int ew, int voff_in_entry, const float* __restrict__ bias, int bias_len,
                               int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ int64_t smem64[];
    int64_t* v_off = smem64;                            // [kAttnThreads]
    float* probs = reinterpret_cast<float*>(v_off + kAttnThreads);   // [kAttnThreads]
    float* scratch = probs + kAttnThreads;              // [32]
    float* qs = scratch + 32;                           // [hd]

    const int64_t t = blockIdx.x;
    const int h = blockIdx.y;
    const int kvh = h / (H / KV);
    const int tid = threadIdx.x;
    const int seq = seq_of_token[t];
    const int p = positions[t];
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int* table = block_tables + static_cast<int64_t>(seq) * table_width;

    for (int e = tid; e < hd; e += kAttnThreads) qs[e] = to_float(q[t * q_stride + h * hd + e]);
    __syncthreads();

    float acc[kMaxDimsPerThread];
#pragma unroll
    for (int i = 0; i < kMaxDimsPerThread; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    const int kept = min(keep_first, lo);               // positions 0..kept-1 lie before the window and stay visible
    for (int run = kept > 0 ? 0 : 1; run < 2; ++run) {
    const int first = run == 0 ? 0 : lo, last = run == 0 ? kept - 1 : p;
    for (int start = first; start <= last; start += kAttnThreads) {
        const int j = start + tid;
        float s = -INFINITY;
        int64_t voff = -1;
        if (j <= last) {
            const int slot = j / page_size;
            int page = slot < table_width ? table[slot] : -1;
            if (page < 0 || page >= num_pages) {
                atomicExch(err, 4);                     // a key this token must see has no page
            } else {
                const int64_t koff = (((static_cast<int64_t>(page) * planes + 0) * KV + kvh) * page_size + j % page_size) * ew;
                voff = (((static_cast<int64_t>(page) * planes + (planes - 1)) * KV + kvh) * page_size + j % page_size) * ew + voff_in_entry;
                const T* kp = cache + koff;
                float d = 0.f;
                for (int e = 0; e < hd; ++e) d = fmaf(qs[e], to_float(kp[e]), d);
                s = d * scale;
                if (bias != nullptr) s += bias[static_cast<int64_t>(h) * bias_len + min(p - j, bias_len - 1)];
            }
        }
        const float tile_max = block_max(s, scratch);
        const float m_new = fmaxf(m, tile_max);
        const float pj = (s == -INFINITY || m_new == -INFINITY) ? 0.f : expf(s - m_new);
        probs[tid] = pj;
        v_off[tid] = voff;
        const float tile_sum = block_sum(pj, scratch);  // also orders the writes above before the reads below
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + tile_sum;
        const int n = min(kAttnThreads, last - start + 1);
#pragma unroll
        for (int i = 0; i < kMaxDimsPerThread; ++i) {
            const int d = tid + i * kAttnThreads;
            if (d < vd) {
                float a = acc[i] * corr;
                for (int jj = 0; jj < n; ++jj) {
                    const int64_t vo = v_off[jj];
                    if (vo >= 0) a = fmaf(probs[jj], to_float(cache[vo + d]), a);
                }
                acc[i] = a;
            }
        }
        m = m_new;
        __syncthreads();
    }
    }
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < kMaxDimsPerThread; ++i) {
        const int d = tid + i * kAttnThreads;
        if (d < vd) out[(t * H + h) * vd + d] = from_float<T>(acc[i] * inv_l);
    }
}

}  // namespace cvb

using namespace cvb;

static int attention_general_launch(void* out, const void* q, const void* cache, const int* block_tables,
                                    int table_width, const int* seq_of_token, const int* positions, int T,
                                    int H, int KV, int hd, int vd, int page_size, int window, int keep_first, int planes,
                                    int q_stride, float scale, int num_pages, int ew, int voff, const float* bias, int bias_len,
                                    int dtype, int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || H <= 0 || KV <= 0 || hd <= 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0)
        return CVB_E_SIZE;
    if (hd > kAttnThreads * kMaxDimsPerThread || vd > kAttnThreads * kMaxDimsPerThread) return CVB_E_SIZE;
    if (H % KV || (planes != 1 && planes != 2) || keep_first < 0 || q_stride < H * hd) return CVB_E_SHAPE;
    if (vd <= 0 || ew < hd || voff < 0 || voff + vd > ew || (planes == 2 && (vd != hd || ew != hd || voff != 0))) return CVB_E_SHAPE;
    if (bias != nullptr && bias_len <= 0) return CVB_E_SHAPE;
    if (H > 65535) return CVB_E_SIZE;
    dim3 grid(static_cast<unsigned>(T), static_cast<unsigned>(H));
    const size_t smem = kAttnThreads * sizeof(int64_t) + (static_cast<size_t>(hd) + kAttnThreads + 32) * sizeof(float);
#define CALL(TY)                                                                                         \
    launch_kernel(paged_attention_general_kernel<TY>, dim3(grid), dim3(kAttnThreads), smem, stream,                             \
        (TY*)out, (const TY*)q, (const TY*)cache, block_tables, table_width, seq_of_token, positions, H, \
        KV, hd, vd, page_size, window, keep_first, planes, q_stride, scale, num_pages, ew, voff, bias, bias_len, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_paged_attention_general(void* out, const void* q, const void* cache, const int* block_tables,
                                           int table_width, const int* seq_of_token, const int* positions, int T,
                                           int H, int KV, int hd, int vd, int page_size, int window, int keep_first, int planes,
                                           int q_stride, float scale, int num_pages, int dtype, int* err_flag,
                                           cudaStream_t stream) {
    if (vd <= 0 || vd > hd) return CVB_E_SHAPE;
    return attention_general_launch(out, q, cache, block_tables, table_width, seq_of_token, positions, T, H, KV, hd, vd, page_size,
                                    window, keep_first, planes, q_stride, scale, num_pages, hd, 0, nullptr, 0, dtype, err_flag, stream);
}

// Entries [key (hd) | value (vd)] per kv head (pages [page, kv head, slot, hd + vd]) and an optional distance table.
extern "C" int cvb_paged_attention_entries(void* out, const void* q, const void* cache, const int* block_tables,
                                           int table_width, const int* seq_of_token, const int* positions, int T,
                                           int H, int KV, int hd, int vd, int page_size, int window, int q_stride, float scale,
                                           int num_pages, const float* bias, int bias_len, int dtype, int* err_flag,
                                           cudaStream_t stream) {
    return attention_general_launch(out, q, cache, block_tables, table_width, seq_of_token, positions, T, H, KV, hd, vd, page_size,
                                    window, 0, 1, q_stride, scale, num_pages, hd + vd, hd, bias, bias_len, dtype, err_flag, stream);
}
