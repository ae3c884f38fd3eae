// Tensor-core attention over a cache whose entries hold a key and, behind it, its value (pages [kv head][slot][dk + dv],
// bf16), with a bias per head and distance added to every score.  Prompt portions and decoded tokens alike.
//
//   token at position p sees key j if j <= p
//   s_j = scale * q . k_j + bias[head, min(p - j, L - 1)];   out = sum_j softmax(s)_j v_j
//   scores, maxima, sums and the output accumulator in float
//
// The structure is that of the kernel for keys that are their own values (attention_keys.cu): a block owns 64 query rows
// of one kv head (64 / g tokens of one request times the g query heads of the group), walks the key tiles up to its last
// token, and gathers each tile of 64 entries through the block table with 16-byte cp.async copies into one of two stages.
// Because a key and its value are neighbours in the cache, ONE sweep fetches both: S = Q K^T reads the first dk columns of
// the tile row-wise (ldmatrix), O += P V the dv columns behind them transposed (ldmatrix.trans).  Four warps of 16 rows,
// `mma.sync.m16n8k16` in bf16 with float accumulation, the softmax online in base 2.  The bias is read from a table
// [H, L] by distance; a tile that lies wholly beyond the table's last distance takes that one entry for all its keys.
// dk and dv are run-time sizes (multiples of 16); the template parameter W bounds both and sizes the register arrays.
// Rows are padded by 16 bytes, which keeps every ldmatrix conflict-free.
#include "common.cuh"
#include "sm100.cuh"
#include "mma_tiles.cuh"

namespace cvb {

constexpr int kBiasTileKeys = 64;
constexpr int kBiasTileRows = 64;
constexpr int kBiasThreads = 128;
constexpr int kBiasDecKeys = 32;                        // keys per tile of the decode form
constexpr float kLog2eBias = 1.4426950408889634f;

struct BiasAttnParams {
    __nv_bfloat16* out;                 // [T, H * dv]
    const __nv_bfloat16* q;             // rows of q_stride elements; the first H * dk of a row are the queries
    const __nv_bfloat16* pages;         // [num_pages, G, page_size, dk + dv]
    const float* bias;                  // [H, L]
    const int* block_tables;            // [S, table_width]
    const int* cu_seqlens;              // [S + 1]
    const int* positions;               // [T]
    int q_stride, table_width, S, H, G, dk, dv, page_size, page_shift, num_pages, L;
    // decode form only: the key tiles of a (request, kv head) are shared out among `splits` blocks (gridDim.z); with more
    // than one, a block leaves its part (unnormalised rows, maxima, sums) in `parts` and a second kernel merges them
    int splits;
    float* parts;                       // [S, G, splits, 16, dv + 2]
    float scale_log2;                   // scale * log2(e)
    int* err;
};

// floats per row of a block's table of biases: tok_per_tile + 63 distances and one more for the odd parity, even, and
// = 4 mod 16 so that the rows of neighbouring heads fall on different banks
__host__ __device__ __forceinline__ int bias_row_floats(int tok_per_tile) {
    const int need = tok_per_tile + kBiasTileKeys;
    return need + ((4 - need % 16) + 16) % 16;
}

__device__ __forceinline__ void bias_page_of(const BiasAttnParams& p, int j, int& slot, int& off) {
    if (p.page_shift >= 0) { slot = j >> p.page_shift; off = j & (p.page_size - 1); }
    else { slot = j / p.page_size; off = j - slot * p.page_size; }
}

// EXACT: dk = dv = W, known to the compiler (no run-time bounds inside the unrolled loops, constant strides)
template <int W, bool EXACT>
__global__ void __launch_bounds__(kBiasThreads, W <= 64 ? 3 : 2)
attn_bias_kernel(const BiasAttnParams p) {
    pdl_trigger();
    pdl_wait();
    const int dk = EXACT ? W : p.dk, dv = EXACT ? W : p.dv;
    const int E = dk + dv;
    const int LDQ = dk + 8, LD = E + 8;                   // padded rows, in elements
    const int CQ = dk >> 3, CE = E >> 3;                  // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sK = sQ + kBiasTileRows * LDQ;         // two stages of kBiasTileKeys * LD
    float* sB = reinterpret_cast<float*>(sK + 2 * kBiasTileKeys * LD);   // the tile's biases: [g][2][XS], see stage_bias

    const int g = p.H / p.G;
    const int tok_per_tile = kBiasTileRows / g;
    const int XS = bias_row_floats(tok_per_tile);
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
    const int n_tiles = key_hi / kBiasTileKeys + 1;

    for (int i = threadIdx.x; i < kBiasTileRows * CQ; i += kBiasThreads) {
        const int r = i / CQ, c = i - r * CQ;
        const int tok = r / g;
        const bool valid = tok < n_tok;
        const __nv_bfloat16* src = valid ? p.q + static_cast<int64_t>(cu0 + q0 + tok) * p.q_stride + (kvh * g + r % g) * dk + c * 8 : p.q;
        cp_async16(sQ + r * LDQ + c * 8, src, valid);
    }

    // a thread's chunks of a tile: chunk i = threadIdx.x + n * kBiasThreads is row i / CE, column i % CE, kept by increments
    const int ld_r0 = threadIdx.x / CE, ld_c0 = threadIdx.x - ld_r0 * CE;
    const int ld_dr = kBiasThreads / CE, ld_dc = kBiasThreads - ld_dr * CE;
    auto load_tile = [&](int it, int stage) {
        const int key0 = it * kBiasTileKeys;
        __nv_bfloat16* dst = sK + stage * kBiasTileKeys * LD;
        int last_slot = -1, page = -1;                    // a thread's rows ascend: the block table is read once per page
        int r = ld_r0, c = ld_c0;
        for (; r < kBiasTileKeys; r += ld_dr, c += ld_dc) {
            if (c >= CE) { c -= CE; ++r; if (r >= kBiasTileKeys) break; }
            const int j = key0 + r;
            bool need = j <= key_hi;
            const __nv_bfloat16* src = p.pages;
            if (need) {
                int slot, off;
                bias_page_of(p, j, slot, off);
                if (slot != last_slot) { page = slot < p.table_width ? table[slot] : -1; last_slot = slot; }
                if (page < 0 || page >= p.num_pages) {
                    atomicExch(p.err, 4);                 // a key a token of this block must see has no page
                    need = false;
                } else {
                    src = p.pages + ((static_cast<int64_t>(page) * p.G + kvh) * p.page_size + off) * E + c * 8;
                }
            }
            cp_async16(dst + r * LD + c * 8, src, need);
        }
    };

    load_tile(0, 0);
    cp_async_commit();

    // the two rows this thread owns in its warp's slab of 16: their positions and their heads' rows of the bias table
    // and where they read the tile's biases: the pair of neighbouring keys (j, j + 1) of score tile nt at tb[half][nt * 4]
    const float2* tb[2];
    float bfar[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + (lane >> 2) + half * 8;
        const int tok = min(r / g, tok_per_tile - 1);     // rows past the block's tokens are never stored
        const int a = tok_per_tile - 1 - tok;
        tb[half] = reinterpret_cast<const float2*>(sB + ((r % g) * 2 + (a & 1)) * XS + (a & ~1) + ((lane & 3) << 1));
        bfar[half] = p.bias[static_cast<int64_t>(kvh * g + r % g) * p.L + p.L - 1] * kLog2eBias;
    }
    const bool warp_has_rows = warp * 16 < n_tok * g;
    const int warp_last_pos = pos_first + min(n_tok - 1, (warp * 16 + 15) / g);
    // The biases of a tile, by distance, once per block: row (head h, parity par) holds at y the bias of x = y + par, which
    // stands for the distance d = (pos_first + tok_per_tile - 1 - key0) - x: bias[h][min(d, L - 1)] * log2(e), or -inf where
    // d < 0 (the key lies behind the token), so that adding it is the causal mask as well.  Token tok of the block and key
    // key0 + c meet at x = (tok_per_tile - 1 - tok) + c; the two parities make every pair (x, x + 1) an aligned 8 bytes.
    auto stage_bias = [&](int key0) {
        const int d0 = pos_first + tok_per_tile - 1 - key0;
        int h = threadIdx.x / (2 * XS), y = threadIdx.x - h * 2 * XS;
        const int dh = kBiasThreads / (2 * XS), dy = kBiasThreads - dh * 2 * XS;
        for (; h < g; h += dh, y += dy) {
            if (y >= 2 * XS) { y -= 2 * XS; ++h; if (h >= g) break; }
            const int par = y >= XS ? 1 : 0;
            const int d = d0 - (y - par * XS + par);
            sB[h * 2 * XS + y] = d < 0 ? -INFINITY : __ldg(p.bias + static_cast<int64_t>(kvh * g + h) * p.L + min(d, p.L - 1)) * kLog2eBias;
        }
    };

    float o[W / 8][4];
#pragma unroll
    for (int dt = 0; dt < W / 8; ++dt) { o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    uint32_t qf[W / 16][4];

    for (int it = 0; it < n_tiles; ++it) {
        if (it + 1 < n_tiles) load_tile(it + 1, (it + 1) & 1);
        cp_async_commit();
        const int key0 = it * kBiasTileKeys;
        const bool all_far = pos_first - (key0 + kBiasTileKeys - 1) >= p.L - 1;   // every key of the tile beyond the table, for every token
        if (!all_far) stage_bias(key0);
        cp_async_wait<1>();                               // everything but the newest group: the query tile and tile `it`
        __syncthreads();
        if (it == 0) {
#pragma unroll
            for (int ks = 0; ks < W / 16; ++ks) {
                if (!EXACT && ks * 16 >= dk) break;
                ldm_x4(qf[ks], sQ + (warp * 16 + (lane & 15)) * LDQ + ks * 16 + (lane >> 4) * 8);
            }
        }
        if (warp_has_rows && key0 <= warp_last_pos) {
            const __nv_bfloat16* tile = sK + (it & 1) * kBiasTileKeys * LD;
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
            // scale, bias (which is the mask too), running maximum and sum
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                float2 b0, b1;
                if (all_far) { b0.x = b0.y = bfar[0]; b1.x = b1.y = bfar[1]; }
                else { b0 = tb[0][nt * 4]; b1 = tb[1][nt * 4]; }
                s[nt][0] = fmaf(s[nt][0], p.scale_log2, b0.x);
                s[nt][1] = fmaf(s[nt][1], p.scale_log2, b0.y);
                s[nt][2] = fmaf(s[nt][2], p.scale_log2, b1.x);
                s[nt][3] = fmaf(s[nt][3], p.scale_log2, b1.y);
                mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
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
        const float inv = l[half] > 0.f ? 1.f / l[half] : 0.f;
        __nv_bfloat16* dst = p.out + (static_cast<int64_t>(cu0 + q0 + tok) * p.H + kvh * g + r % g) * dv;
#pragma unroll
        for (int dt = 0; dt < W / 8; ++dt) {
            const int d = dt * 8 + ((lane & 3) << 1);
            if (!EXACT && d >= dv) break;
            *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(o[dt][half * 2] * inv, o[dt][half * 2 + 1] * inv);
        }
    }
}

// ---- decoded tokens: one token per request ---------------------------------------------------------------------------
//
// A block owns one (request, kv head): the g <= 16 query heads of the group are the rows of ONE 16-row slab, and each of
// the block's warps takes every n-th key tile (32 entries) for itself: it fetches its tiles into two stages of its own
// (cp.async by its own lanes, __syncwarp, no block-wide barrier in the loop), keeps its own running maximum, sum and
// accumulator, and the warps' partial results are merged through shared memory at the end.  Eight warps, or as many
// as have room for their stages where the entries are wide (six at 128 + 128 elements).  When few (request, kv head) pairs would leave SMs
// idle, the tiles are shared out among `splits` blocks as well, which leave their parts in scratch for a merge kernel.
template <int W, bool EXACT>
__global__ void __launch_bounds__(256)
attn_bias_decode_kernel(const BiasAttnParams p) {
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
    float* red_ml = reinterpret_cast<float*>(sK + nw * 2 * kBiasDecKeys * LD);         // [warps][16][2]
    const int g = p.H / p.G;
    const int seq = blockIdx.x, kvh = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = p.cu_seqlens[seq];
    const int pos = p.positions[t];
    const int* table = p.block_tables + static_cast<int64_t>(seq) * p.table_width;
    const int n_tiles = pos / kBiasDecKeys + 1;

    for (int i = threadIdx.x; i < 16 * CQ; i += blockDim.x) {
        const int r = i / CQ, c = i - r * CQ;
        const bool valid = r < g;
        cp_async16(sQ + r * LDQ + c * 8, valid ? p.q + static_cast<int64_t>(t) * p.q_stride + (kvh * g + r) * dk + c * 8 : p.q, valid);
    }
    cp_async_commit();

    __nv_bfloat16* my = sK + warp * 2 * kBiasDecKeys * LD;
    const int ld_r0 = lane / CE, ld_c0 = lane - ld_r0 * CE;
    const int ld_dr = 32 / CE, ld_dc = 32 - ld_dr * CE;
    auto load_tile = [&](int it, int stage) {
        const int key0 = it * kBiasDecKeys;
        __nv_bfloat16* dst = my + stage * kBiasDecKeys * LD;
        int last_slot = -1, page = -1;
        const __nv_bfloat16* page_base = p.pages;
        int r = ld_r0, c = ld_c0;                         // chunk lane + 32 n is row (lane + 32 n) / CE: kept by increments
        if (p.page_shift >= 5) {
            // pages of 32 tokens and more (a power of two): the tile lies in ONE page, its rows side by side
            const int slot = key0 >> p.page_shift;
            page = slot < p.table_width ? table[slot] : -1;
            const bool ok = page >= 0 && page < p.num_pages;
            if (!ok) atomicExch(p.err, 4);
            const __nv_bfloat16* base = ok ? p.pages + ((static_cast<int64_t>(page) * p.G + kvh) * p.page_size + (key0 & (p.page_size - 1))) * E
                                           : p.pages;
            const int live = ok ? pos - key0 : -1;        // rows 0..live hold keys the token sees
            for (; r < kBiasDecKeys; r += ld_dr, c += ld_dc) {
                if (c >= CE) { c -= CE; ++r; if (r >= kBiasDecKeys) break; }
                const bool need = r <= live;
                cp_async16(dst + r * LD + c * 8, need ? base + r * E + c * 8 : p.pages, need);
            }
            return;
        }
        for (; r < kBiasDecKeys; r += ld_dr, c += ld_dc) {
            if (c >= CE) { c -= CE; ++r; if (r >= kBiasDecKeys) break; }
            const int j = key0 + r;
            bool need = j <= pos;
            const __nv_bfloat16* src = p.pages;
            if (need) {
                int slot, off;
                bias_page_of(p, j, slot, off);
                if (slot != last_slot) {
                    page = slot < p.table_width ? table[slot] : -1;
                    last_slot = slot;
                    page_base = p.pages + (static_cast<int64_t>(page) * p.G + kvh) * p.page_size * E;
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
    const float* brow[2];
    float bfar[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = min((lane >> 2) + half * 8, g - 1);   // rows past the group repeat its last head; never stored
        brow[half] = p.bias + static_cast<int64_t>(kvh * g + r) * p.L;
        bfar[half] = brow[half][p.L - 1] * kLog2eBias;
    }

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
        const int key0 = it * kBiasDecKeys;
        const __nv_bfloat16* tile = my + (n & 1) * kBiasDecKeys * LD;
        float s[kBiasDecKeys / 8][4];
#pragma unroll
        for (int nt = 0; nt < kBiasDecKeys / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < W / 16; ++ks) {
            if (!EXACT && ks * 16 >= dk) break;
#pragma unroll
            for (int np = 0; np < kBiasDecKeys / 16; ++np) {
                uint32_t b[4];
                ldm_x4(b, tile + (np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_16816(s[np * 2], qf[ks], b[0], b[1]);
                mma_16816(s[np * 2 + 1], qf[ks], b[2], b[3]);
            }
        }
        const bool all_far = pos - (key0 + kBiasDecKeys - 1) >= p.L - 1;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < kBiasDecKeys / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int half = e >> 1;
                const int j = key0 + nt * 8 + ((lane & 3) << 1) + (e & 1);
                const int dist = pos - j;
                float v = -INFINITY;
                if (dist >= 0) {
                    const float b = (all_far || dist >= p.L - 1) ? bfar[half] : __ldg(brow[half] + dist) * kLog2eBias;
                    v = fmaf(s[nt][e], p.scale_log2, b);
                }
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
        for (int nt = 0; nt < kBiasDecKeys / 8; ++nt) {
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
        for (int kk = 0; kk < kBiasDecKeys / 16; ++kk) {
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
            acc += reinterpret_cast<const float*>(sK + w * 2 * kBiasDecKeys * LD)[r * dv + d] * f;
        }
        if (p.splits == 1) {
            p.out[(static_cast<int64_t>(t) * p.H + kvh * g + r) * dv + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
        } else {
            float* dst = p.parts + ((static_cast<int64_t>(seq) * p.G + kvh) * p.splits + blockIdx.z) * 16 * (dv + 2) + r * (dv + 2);
            dst[d] = acc;
            if (d == 0) { dst[dv] = mm; dst[dv + 1] = ll; }
        }
    }
}

// out = the parts of a (request, kv head) added up: rows scaled to the common maximum, divided by the common sum
__global__ void attn_bias_merge_kernel(const BiasAttnParams p) {
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
        p.out[(static_cast<int64_t>(t) * p.H + kvh * g + r) * dv + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
    }
}

template <int W, bool EXACT>
int launch_attn_bias_decode(const BiasAttnParams& p, cudaStream_t stream) {
    const int E = p.dk + p.dv;
    // as many warps as their stages leave room for, eight at most
    const size_t per_warp = static_cast<size_t>(2) * kBiasDecKeys * (E + 8) * sizeof(__nv_bfloat16) + 16 * 2 * sizeof(float);
    const size_t room = 216 * 1024 - static_cast<size_t>(16) * (p.dk + 8) * sizeof(__nv_bfloat16);
    const int nw = room / per_warp >= 8 ? 8 : static_cast<int>(room / per_warp);
    const size_t smem = (static_cast<size_t>(16) * (p.dk + 8) + static_cast<size_t>(nw) * 2 * kBiasDecKeys * (E + 8)) * sizeof(__nv_bfloat16)
                        + nw * 16 * 2 * sizeof(float);
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(attn_bias_decode_kernel<W, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024) != cudaSuccess)
            return launch_status();
        raised = true;
    }
    launch_kernel(attn_bias_decode_kernel<W, EXACT>, dim3(p.S, p.G, p.splits), dim3(nw * 32), smem, stream, p);
    if (p.splits > 1) launch_kernel(attn_bias_merge_kernel, dim3(p.S, p.G, (p.H / p.G * p.dv + 127) / 128), dim3(128), 0, stream, p);
    return launch_status();
}

template <int W, bool EXACT>
int launch_attn_bias(const BiasAttnParams& p, int num_tiles, cudaStream_t stream) {
    const int E = p.dk + p.dv;
    const int g = p.H / p.G;
    const size_t smem = (static_cast<size_t>(kBiasTileRows) * (p.dk + 8) + static_cast<size_t>(2) * kBiasTileKeys * (E + 8)) * sizeof(__nv_bfloat16)
                        + static_cast<size_t>(g) * 2 * bias_row_floats(kBiasTileRows / g) * sizeof(float);
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(attn_bias_kernel<W, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 136 * 1024) != cudaSuccess)
            return launch_status();
        raised = true;
    }
    launch_kernel(attn_bias_kernel<W, EXACT>, dim3(num_tiles, p.G), dim3(kBiasThreads), smem, stream, p);
    return launch_status();
}

}  // namespace cvb

using namespace cvb;

// 1 if the kernel takes this shape: bf16, key and value sizes 16..128 in steps of 16, up to 64 query heads per kv head.
extern "C" int cvb_attn_bias_supported(int H, int G, int dk, int dv) {
    return (H > 0 && G > 0 && H % G == 0 && H / G <= kBiasTileRows && dk >= 16 && dk <= 128 && dk % 16 == 0
            && dv >= 16 && dv <= 128 && dv % 16 == 0) ? 1 : 0;
}

extern "C" int cvb_attn_bias_bf16(void* out, const void* q, int q_stride, const void* pages, const int* block_tables,
                                  int table_width, const int* cu_seqlens, const int* positions, int S, int num_tiles, int H,
                                  int G, int dk, int dv, int page_size, float scale, const float* bias, int bias_len,
                                  int num_pages, int all_single, int splits, float* parts, int64_t parts_floats, int* err_flag,
                                  cudaStream_t stream) {
    if (num_tiles == 0 || S == 0) return CVB_OK;
    if (S < 0 || num_tiles < 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0 || bias_len <= 0 || bias == nullptr) return CVB_E_SIZE;
    if (!cvb_attn_bias_supported(H, G, dk, dv)) return CVB_E_UNSUPPORTED;
    if (q_stride < H * dk || q_stride % 8 != 0) return CVB_E_ALIGN;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(pages) | reinterpret_cast<uintptr_t>(out)) & 15) return CVB_E_ALIGN;
    if (G > 65535) return CVB_E_SIZE;
    BiasAttnParams p;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.pages = static_cast<const __nv_bfloat16*>(pages);
    p.bias = bias; p.L = bias_len;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.q_stride = q_stride; p.table_width = table_width; p.S = S; p.H = H; p.G = G; p.dk = dk; p.dv = dv; p.page_size = page_size;
    p.num_pages = num_pages;
    p.page_shift = -1;
    for (int sh = 0; sh < 31; ++sh)
        if ((1 << sh) == page_size) p.page_shift = sh;
    p.scale_log2 = scale * kLog2eBias;
    p.err = err_flag;
    p.splits = 1; p.parts = nullptr;
    const bool decode = all_single && H / G <= 16;        // every request brings one token: the kernel for decoded tokens
    if (decode && splits > 1) {
        if (splits > 64) return CVB_E_SIZE;
        if (parts == nullptr || parts_floats < static_cast<int64_t>(S) * G * splits * 16 * (dv + 2)) return CVB_E_SCRATCH;
        p.splits = splits; p.parts = parts;
    }
    const int w = dk > dv ? dk : dv;
    const bool exact = dk == dv && (dk == 32 || dk == 64 || dk == 96 || dk == 128);
#define CVB_BIAS_WIDTH(WW)                                                                                               \
    if (w <= WW) {                                                                                                       \
        if (decode) return exact ? launch_attn_bias_decode<WW, true>(p, stream) : launch_attn_bias_decode<WW, false>(p, stream); \
        return exact ? launch_attn_bias<WW, true>(p, num_tiles, stream) : launch_attn_bias<WW, false>(p, num_tiles, stream);     \
    }
    CVB_BIAS_WIDTH(32)
    CVB_BIAS_WIDTH(64)
    CVB_BIAS_WIDTH(96)
    CVB_BIAS_WIDTH(128)
#undef CVB_BIAS_WIDTH
    return CVB_E_UNSUPPORTED;
}
