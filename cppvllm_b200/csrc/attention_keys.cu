// Tensor-core attention over a cache of keys that are also the values (pages [kv head][slot][HD], bf16), behind a
// sliding window that keeps the sequence's first positions visible.  Prompt portions and decoded tokens alike.
//
//   token at position p of a request sees key j if  j <= p  and  (window == 0  or  p - j < window  or  j < keep_first)
//   s_j = scale * q . k_j;   out = sum_j softmax(s)_j k_j          scores, maxima, sums and the output accumulator in float
//
// A block owns 64 query rows of one kv head: 64 / g tokens of one request times the g query heads of the group (row r is
// token r / g, head r % g), so a key tile is read once for the whole group.  It walks the key tiles that hold a kept first
// position and lie wholly before the window, then the tiles of the window up to the block's last token; a tile is 64 keys,
// gathered row by row through the block table with 16-byte cp.async copies into one of two stages (rows that no token of
// the block may see are zero-filled instead, so that pages the window has given back are never touched).  Because the
// values are the keys, ONE tile in shared memory feeds both products: S = Q K^T reads it row-wise (ldmatrix), O += P K
// reads it transposed (ldmatrix.trans); a cache with separate values would move twice the bytes.  Four warps, each 16
// rows: `mma.sync.m16n8k16` in bf16 with float accumulation, the softmax online in base 2.  Rows are padded by 16 bytes,
// which makes every ldmatrix conflict-free for all head sizes that are multiples of 16.
// The value may be narrower than the key (`vd` <= HD, a multiple of 16): only the first vd elements of a key are its value
// (a latent vector with a positional part behind it); O += P K then stops at column vd and the output rows are [T, H, vd].
#include "common.cuh"
#include "sm100.cuh"
#include "mma_tiles.cuh"

namespace cvb {

constexpr int kTileKeys = 64;
constexpr int kTileRows = 64;
constexpr int kKeysThreads = 128;
constexpr float kLog2eKeys = 1.4426950408889634f;

struct KeysAttnParams {
    __nv_bfloat16* out;                 // [T, H * HD]
    const __nv_bfloat16* q;             // rows of q_stride elements; the first H * HD of a row are the queries
    const __nv_bfloat16* pages;         // [num_pages, KV, page_size, HD]
    const int* block_tables;            // [S, table_width]
    const int* cu_seqlens;              // [S + 1]
    const int* positions;               // [T]
    int q_stride, table_width, S, H, KV, page_size, window, keep_first, num_pages;
    int vd;                             // leading elements of a key that are its value (HD: all of them)
    int kv_phys;                        // kv heads the pages hold; KV (the heads the grid walks) is a multiple of it: the
                                        // query heads of one stored kv head may be dealt with as several groups
    int page_shift;                     // log2(page_size) if that is a power of two, else -1
    // decode form only: the key tiles of a (request, kv head) are shared out among `splits` blocks (gridDim.z); with more
    // than one, a block leaves its part (unnormalised rows, maxima, sums) in `parts` and a second kernel merges them
    int splits;
    float* parts;                       // [S, KV, splits, 16, HD + 2]
    float scale_log2;                   // scale * log2(e)
    int* err;
};

// page and offset of key j
__device__ __forceinline__ void page_of(const KeysAttnParams& p, int j, int& slot, int& off) {
    if (p.page_shift >= 0) { slot = j >> p.page_shift; off = j & (p.page_size - 1); }
    else { slot = j / p.page_size; off = j - slot * p.page_size; }
}
template <int HD>
__global__ void __launch_bounds__(kKeysThreads, 3)
attn_keys_kernel(const KeysAttnParams p) {
    pdl_trigger();
    pdl_wait();
    constexpr int LD = HD + 8;                            // padded row, in elements
    constexpr int CPR = HD / 8;                           // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sK = sQ + kTileRows * LD;              // two stages of kTileKeys * LD

    const int g = p.H / p.KV;
    const int tok_per_tile = kTileRows / g;
    const int kvh = blockIdx.y;
    const int kvp = kvh / (p.KV / p.kv_phys);             // the kv head as the pages hold it
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
    const int key_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int keep = p.window > 0 ? p.keep_first : 0;
    const int first_tile = key_lo / kTileKeys;
    const int n_win = key_hi / kTileKeys - first_tile + 1;
    const int n_kept = keep > 0 ? min((keep - 1) / kTileKeys + 1, first_tile) : 0;   // tiles wholly before the window's
    const int n_tiles = n_kept + n_win;

    // the query tile
    for (int i = threadIdx.x; i < kTileRows * CPR; i += kKeysThreads) {
        const int r = i / CPR, c = i - r * CPR;
        const int tok = r / g;
        const bool valid = tok < n_tok;
        const __nv_bfloat16* src = valid ? p.q + static_cast<int64_t>(cu0 + q0 + tok) * p.q_stride + (kvh * g + r % g) * HD + c * 8 : p.q;
        cp_async16(sQ + r * LD + c * 8, src, valid);
    }

    auto load_tile = [&](int it, int stage) {
        const int key0 = (it < n_kept ? it : first_tile + it - n_kept) * kTileKeys;
        __nv_bfloat16* dst = sK + stage * kTileKeys * LD;
        int last_slot = -1, page = -1;                    // a thread's rows ascend: the block table is read once per page
        for (int i = threadIdx.x; i < kTileKeys * CPR; i += kKeysThreads) {
            const int r = i / CPR, c = i - r * CPR;
            const int j = key0 + r;
            bool need = j <= key_hi && (j >= key_lo || j < keep);
            const __nv_bfloat16* src = p.pages;
            if (need) {
                int slot, off;
                page_of(p, j, slot, off);
                if (slot != last_slot) { page = slot < p.table_width ? table[slot] : -1; last_slot = slot; }
                if (page < 0 || page >= p.num_pages) {
                    atomicExch(p.err, 4);                 // a key a token of this block must see has no page
                    need = false;
                } else {
                    src = p.pages + ((static_cast<int64_t>(page) * p.kv_phys + kvp) * p.page_size + off) * HD + c * 8;
                }
            }
            cp_async16(dst + r * LD + c * 8, src, need);
        }
    };

    load_tile(0, 0);
    cp_async_commit();

    // the two rows this thread owns in its warp's slab of 16
    int row_lo[2], row_hi[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + (lane >> 2) + half * 8;
        const int tok = min(r / g, n_tok - 1);            // rows past the block's tokens repeat the last one; never stored
        row_hi[half] = pos_first + tok;
        row_lo[half] = p.window > 0 ? max(0, row_hi[half] - p.window + 1) : 0;
    }
    const bool warp_has_rows = warp * 16 < n_tok * g;
    const int warp_last_pos = pos_first + min(n_tok - 1, (warp * 16 + 15) / g);
    const int warp_first_pos = pos_first + min(n_tok - 1, (warp * 16) / g);
    const int warp_min_lo = p.window > 0 ? max(0, warp_first_pos - p.window + 1) : 0;

    float o[HD / 8][4];
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) { o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    uint32_t qf[HD / 16][4];

    for (int it = 0; it < n_tiles; ++it) {
        if (it + 1 < n_tiles) load_tile(it + 1, (it + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();                               // everything but the newest group: the query tile and tile `it`
        __syncthreads();
        if (it == 0) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
                ldm_x4(qf[ks], sQ + (warp * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8);
        }
        const int key0 = (it < n_kept ? it : first_tile + it - n_kept) * kTileKeys;
        const bool touches = key0 <= warp_last_pos && (key0 + kTileKeys > warp_min_lo || key0 < keep);
        if (warp_has_rows && touches) {
            const __nv_bfloat16* tile = sK + (it & 1) * kTileKeys * LD;
            float s[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b[4];
                    ldm_x4(b, tile + (np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
                    mma_16816(s[np * 2], qf[ks], b[0], b[1]);
                    mma_16816(s[np * 2 + 1], qf[ks], b[2], b[3]);
                }
            }
            // mask, running maximum and sum
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int half = e >> 1;
                    const int j = key0 + nt * 8 + ((lane & 3) << 1) + (e & 1);
                    const bool sees = j <= row_hi[half] && (j >= row_lo[half] || j < keep);
                    const float v = sees ? s[nt][e] * p.scale_log2 : -INFINITY;
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
            for (int dt = 0; dt < HD / 8; ++dt) {
                o[dt][0] *= corr[0]; o[dt][1] *= corr[0]; o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
            }
            // O += P K: the same tile, read transposed
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t a[4];
                a[0] = pack2(s[kk * 2][0], s[kk * 2][1]);
                a[1] = pack2(s[kk * 2][2], s[kk * 2][3]);
                a[2] = pack2(s[kk * 2 + 1][0], s[kk * 2 + 1][1]);
                a[3] = pack2(s[kk * 2 + 1][2], s[kk * 2 + 1][3]);
#pragma unroll
                for (int dp = 0; dp < HD / 16; ++dp) {
                    if (dp * 16 >= p.vd) break;
                    uint32_t b[4];
                    ldm_x4_trans(b, tile + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dp * 16 + ((lane >> 4) & 1) * 8);
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
        const float inv = l[half] > 0.f ? 1.f / l[half] : 0.f;
        __nv_bfloat16* dst = p.out + (static_cast<int64_t>(cu0 + q0 + tok) * p.H + kvh * g + r % g) * p.vd;
#pragma unroll
        for (int dt = 0; dt < HD / 8; ++dt) {
            const int d = dt * 8 + ((lane & 3) << 1);
            if (d >= p.vd) break;
            *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(o[dt][half * 2] * inv, o[dt][half * 2 + 1] * inv);
        }
    }
}

// ---- decoded tokens: one token per request ---------------------------------------------------------------------------
//
// A block owns one (request, kv head): the g <= 16 query heads of the group are the rows of ONE 16-row slab, so the eight
// warps have nothing to share but the keys, and each takes every eighth key tile (32 keys) for itself: it fetches its tiles
// into two stages of its own (cp.async by its own lanes, __syncwarp, no block-wide barrier in the loop), keeps its own
// running maximum, sum and accumulator, and the eight partial results are merged through shared memory at the end.  Up to
// sixteen tiles are in flight per block.  When few (request, kv head) pairs would leave SMs idle, the tiles are shared out
// among `splits` blocks as well, which leave their parts in scratch for a small merge kernel.  Eight warps of short tiles rather than four of long ones: with one warp per
// scheduler every instruction's latency shows (measured: 14 k instructions a warp in 90 k cycles, stalled on fixed-latency
// dependencies), two warps per scheduler with half the instructions each overlap.
constexpr int kDecWarps = 8;
constexpr int kDecKeys = 32;                             // keys per tile of the decode form

template <int HD>
__global__ void __launch_bounds__(kDecWarps * 32)
attn_keys_decode_kernel(const KeysAttnParams p) {
    pdl_trigger();
    pdl_wait();
    constexpr int LD = HD + 8;
    constexpr int CPR = HD / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);                    // [16][LD]
    __nv_bfloat16* sK = sQ + 16 * LD;                                                  // [warps][2][64][LD]
    float* red_ml = reinterpret_cast<float*>(sK + kDecWarps * 2 * kDecKeys * LD);     // [warps][16][2]
    const int g = p.H / p.KV;
    const int seq = blockIdx.x, kvh = blockIdx.y;
    const int kvp = kvh / (p.KV / p.kv_phys);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = p.cu_seqlens[seq];
    const int pos = p.positions[t];
    const int* table = p.block_tables + static_cast<int64_t>(seq) * p.table_width;
    const int key_lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int keep = p.window > 0 ? p.keep_first : 0;
    const int first_tile = key_lo / kDecKeys;
    const int n_win = pos / kDecKeys - first_tile + 1;
    const int n_kept = keep > 0 ? min((keep - 1) / kDecKeys + 1, first_tile) : 0;
    const int n_tiles = n_kept + n_win;

    for (int i = threadIdx.x; i < 16 * CPR; i += kDecWarps * 32) {
        const int r = i / CPR, c = i - r * CPR;
        const bool valid = r < g;
        cp_async16(sQ + r * LD + c * 8, valid ? p.q + static_cast<int64_t>(t) * p.q_stride + (kvh * g + r) * HD + c * 8 : p.q, valid);
    }
    cp_async_commit();

    __nv_bfloat16* my = sK + warp * 2 * kDecKeys * LD;
    auto load_tile = [&](int it, int stage) {
        const int key0 = (it < n_kept ? it : first_tile + it - n_kept) * kDecKeys;
        __nv_bfloat16* dst = my + stage * kDecKeys * LD;
        int last_slot = -1, page = -1;
        const __nv_bfloat16* page_base = p.pages;
        // a lane's chunks: with 32 % CPR == 0 the lane keeps its column and walks down the rows
        for (int i = lane; i < kDecKeys * CPR; i += 32) {
            const int r = i / CPR, c = i - r * CPR;
            const int j = key0 + r;
            bool need = j <= pos && (j >= key_lo || j < keep);
            const __nv_bfloat16* src = p.pages;
            if (need) {
                int slot, off;
                page_of(p, j, slot, off);
                if (slot != last_slot) {
                    page = slot < p.table_width ? table[slot] : -1;
                    last_slot = slot;
                    page_base = p.pages + (static_cast<int64_t>(page) * p.kv_phys + kvp) * p.page_size * HD;
                }
                if (page < 0 || page >= p.num_pages) {
                    atomicExch(p.err, 4);
                    need = false;
                } else {
                    src = page_base + off * HD + c * 8;
                }
            }
            cp_async16(dst + r * LD + c * 8, src, need);
        }
    };

    const int lanes_w = kDecWarps * p.splits;             // warps that share the tiles: this block's and its siblings'
    const int gw = blockIdx.z * kDecWarps + warp;
    const int my_tiles = n_tiles > gw ? (n_tiles - gw + lanes_w - 1) / lanes_w : 0;     // tiles gw, gw + lanes_w, ...
    if (my_tiles > 0) load_tile(gw, 0);
    cp_async_commit();
    cp_async_wait<1>();                                   // this thread's share of the queries
    __syncthreads();                                      // everybody's share
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) ldm_x4(qf[ks], sQ + (lane & 15) * LD + ks * 16 + (lane >> 4) * 8);

    float o[HD / 8][4];
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) { o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int n = 0; n < my_tiles; ++n) {
        const int it = gw + n * lanes_w;
        if (n + 1 < my_tiles) load_tile(it + lanes_w, (n + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();
        const int key0 = (it < n_kept ? it : first_tile + it - n_kept) * kDecKeys;
        const __nv_bfloat16* tile = my + (n & 1) * kDecKeys * LD;
        float s[kDecKeys / 8][4];
#pragma unroll
        for (int nt = 0; nt < kDecKeys / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < kDecKeys / 16; ++np) {
                uint32_t b[4];
                ldm_x4(b, tile + (np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_16816(s[np * 2], qf[ks], b[0], b[1]);
                mma_16816(s[np * 2 + 1], qf[ks], b[2], b[3]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < kDecKeys / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = key0 + nt * 8 + ((lane & 3) << 1) + (e & 1);
                const bool sees = j <= pos && (j >= key_lo || j < keep);
                const float v = sees ? s[nt][e] * p.scale_log2 : -INFINITY;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
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
        for (int nt = 0; nt < kDecKeys / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pj = (s[nt][e] == -INFINITY) ? 0.f : ex2(s[nt][e] - m[e >> 1]);
                s[nt][e] = pj;
                sum[e >> 1] += pj;
            }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) l[half] = l[half] * corr[half] + sum[half];
#pragma unroll
        for (int dt = 0; dt < HD / 8; ++dt) {
            o[dt][0] *= corr[0]; o[dt][1] *= corr[0]; o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < kDecKeys / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack2(s[kk * 2][0], s[kk * 2][1]);
            a[1] = pack2(s[kk * 2][2], s[kk * 2][3]);
            a[2] = pack2(s[kk * 2 + 1][0], s[kk * 2 + 1][1]);
            a[3] = pack2(s[kk * 2 + 1][2], s[kk * 2 + 1][3]);
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                if (dp * 16 >= p.vd) break;
                uint32_t b[4];
                ldm_x4_trans(b, tile + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dp * 16 + ((lane >> 4) & 1) * 8);
                mma_16816(o[dp * 2], a, b[0], b[1]);
                mma_16816(o[dp * 2 + 1], a, b[2], b[3]);
            }
        }
        __syncwarp();                                     // the stage may be filled again
    }
    cp_async_wait<0>();

    // merge the warps' parts: each leaves its sums, maxima and its accumulator [16][HD] (float) in its own stages
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 1);
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 2);
    }
    __syncwarp();
    float* part = reinterpret_cast<float*>(my);            // 16 * HD floats = 64 * HD bytes, within the warp's two stages (2 * 32 * LD * 2)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = (lane >> 2) + half * 8;
        if ((lane & 3) == 0) { red_ml[(warp * 16 + r) * 2] = m[half]; red_ml[(warp * 16 + r) * 2 + 1] = l[half]; }
#pragma unroll
        for (int dt = 0; dt < HD / 8; ++dt) {
            const int d = dt * 8 + ((lane & 3) << 1);
            part[r * HD + d] = o[dt][half * 2];
            part[r * HD + d + 1] = o[dt][half * 2 + 1];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < g * HD; i += kDecWarps * 32) {
        const int r = i / HD, d = i - r * HD;
        if (d >= p.vd) continue;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, red_ml[(w * 16 + r) * 2]);
        float ll = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) {
            const float mw = red_ml[(w * 16 + r) * 2];
            const float f = mw == -INFINITY ? 0.f : ex2(mw - mm);
            ll += red_ml[(w * 16 + r) * 2 + 1] * f;
            acc += reinterpret_cast<const float*>(sK + w * 2 * kDecKeys * LD)[r * HD + d] * f;
        }
        if (p.splits == 1) {
            p.out[(static_cast<int64_t>(t) * p.H + kvh * g + r) * p.vd + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
        } else {
            float* dst = p.parts + ((static_cast<int64_t>(seq) * p.KV + kvh) * p.splits + blockIdx.z) * 16 * (HD + 2) + r * (HD + 2);
            dst[d] = acc;
            if (d == 0) { dst[HD] = mm; dst[HD + 1] = ll; }
        }
    }
}

// out = the parts of a (request, kv head) added up: rows scaled to the common maximum, divided by the common sum
template <int HD>
__global__ void attn_keys_merge_kernel(const KeysAttnParams p) {
    pdl_trigger();
    pdl_wait();
    const int g = p.H / p.KV;
    const int seq = blockIdx.x, kvh = blockIdx.y;
    const int t = p.cu_seqlens[seq];
    const float* base = p.parts + (static_cast<int64_t>(seq) * p.KV + kvh) * p.splits * 16 * (HD + 2);
    for (int i = blockIdx.z * blockDim.x + threadIdx.x; i < g * HD; i += gridDim.z * blockDim.x) {      // an element a thread
        const int r = i / HD, d = i - r * HD;
        if (d >= p.vd) continue;
        float mm = -INFINITY;
        for (int z = 0; z < p.splits; ++z) mm = fmaxf(mm, base[(z * 16 + r) * (HD + 2) + HD]);
        float ll = 0.f, acc = 0.f;
        for (int z = 0; z < p.splits; ++z) {
            const float* row = base + (z * 16 + r) * (HD + 2);
            const float f = row[HD] == -INFINITY ? 0.f : ex2(row[HD] - mm);
            ll += row[HD + 1] * f;
            acc += row[d] * f;
        }
        p.out[(static_cast<int64_t>(t) * p.H + kvh * g + r) * p.vd + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
    }
}

template <int HD>
int launch_attn_keys_decode(const KeysAttnParams& p, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(16 + kDecWarps * 2 * kDecKeys) * (HD + 8) * sizeof(__nv_bfloat16) + kDecWarps * 16 * 2 * sizeof(float);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        if (cudaFuncSetAttribute(attn_keys_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
            return launch_status();
        raised = true;
    }
    launch_kernel(attn_keys_decode_kernel<HD>, dim3(p.S, p.KV, p.splits), dim3(kDecWarps * 32), smem, stream, p);
    if (p.splits > 1) launch_kernel(attn_keys_merge_kernel<HD>, dim3(p.S, p.KV, (p.H / p.KV * HD + 127) / 128), dim3(128), 0, stream, p);
    return launch_status();
}

template <int HD>
int launch_attn_keys(const KeysAttnParams& p, int num_tiles, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(kTileRows + 2 * kTileKeys) * (HD + 8) * sizeof(__nv_bfloat16);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        if (cudaFuncSetAttribute(attn_keys_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
            return launch_status();
        raised = true;
    }
    launch_kernel(attn_keys_kernel<HD>, dim3(num_tiles, p.KV), dim3(kKeysThreads), smem, stream, p);
    return launch_status();
}

}  // namespace cvb

using namespace cvb;

// 1 if the kernel takes this shape: bf16, head sizes 16..128 in steps of 16, groups of up to 64 query heads per kv head.
extern "C" int cvb_attn_keys_supported(int H, int KV, int hd) {
    return (H > 0 && KV > 0 && H % KV == 0 && H / KV <= kTileRows && hd >= 16 && hd <= 128 && hd % 16 == 0) ? 1 : 0;
}

extern "C" int cvb_attn_keys_bf16(void* out, const void* q, int q_stride, const void* pages, const int* block_tables,
                                  int table_width, const int* cu_seqlens, const int* positions, int S, int num_tiles, int H,
                                  int KV, int hd, int vd, int page_size, int window, int keep_first, float scale, int num_pages,
                                  int all_single, int splits, float* parts, int64_t parts_floats, int kv_phys, int* err_flag,
                                  cudaStream_t stream) {
    if (num_tiles == 0 || S == 0) return CVB_OK;
    if (S < 0 || num_tiles < 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0 || window < 0 || keep_first < 0) return CVB_E_SIZE;
    if (!cvb_attn_keys_supported(H, KV, hd)) return CVB_E_UNSUPPORTED;
    if (vd <= 0 || vd > hd || vd % 16 != 0) return CVB_E_UNSUPPORTED;
    if (kv_phys <= 0) kv_phys = KV;
    if (KV % kv_phys != 0) return CVB_E_SHAPE;
    if (q_stride < H * hd || q_stride % 8 != 0) return CVB_E_ALIGN;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(pages) | reinterpret_cast<uintptr_t>(out)) & 15) return CVB_E_ALIGN;
    if (KV > 65535) return CVB_E_SIZE;
    KeysAttnParams p;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.pages = static_cast<const __nv_bfloat16*>(pages);
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.q_stride = q_stride; p.table_width = table_width; p.S = S; p.H = H; p.KV = KV; p.page_size = page_size;
    p.window = window; p.keep_first = keep_first; p.num_pages = num_pages; p.vd = vd; p.kv_phys = kv_phys;
    p.page_shift = -1;
    for (int sh = 0; sh < 31; ++sh)
        if ((1 << sh) == page_size) p.page_shift = sh;
    p.scale_log2 = scale * kLog2eKeys;
    p.err = err_flag;
    p.splits = 1; p.parts = nullptr;
    if (all_single && H / KV <= 16 && splits > 1) {
        if (splits > 64) return CVB_E_SIZE;
        if (parts == nullptr || parts_floats < static_cast<int64_t>(S) * KV * splits * 16 * (hd + 2)) return CVB_E_SCRATCH;
        p.splits = splits; p.parts = parts;
    }
    if (all_single && H / KV <= 16) {                     // every request brings one token: the kernel for decoded tokens
        switch (hd) {
            case 16: return launch_attn_keys_decode<16>(p, stream);
            case 32: return launch_attn_keys_decode<32>(p, stream);
            case 48: return launch_attn_keys_decode<48>(p, stream);
            case 64: return launch_attn_keys_decode<64>(p, stream);
            case 80: return launch_attn_keys_decode<80>(p, stream);
            case 96: return launch_attn_keys_decode<96>(p, stream);
            case 112: return launch_attn_keys_decode<112>(p, stream);
            case 128: return launch_attn_keys_decode<128>(p, stream);
        }
        return CVB_E_UNSUPPORTED;
    }
    switch (hd) {
        case 16: return launch_attn_keys<16>(p, num_tiles, stream);
        case 32: return launch_attn_keys<32>(p, num_tiles, stream);
        case 48: return launch_attn_keys<48>(p, num_tiles, stream);
        case 64: return launch_attn_keys<64>(p, num_tiles, stream);
        case 80: return launch_attn_keys<80>(p, num_tiles, stream);
        case 96: return launch_attn_keys<96>(p, num_tiles, stream);
        case 112: return launch_attn_keys<112>(p, num_tiles, stream);
        case 128: return launch_attn_keys<128>(p, num_tiles, stream);
    }
    return CVB_E_UNSUPPORTED;
}
