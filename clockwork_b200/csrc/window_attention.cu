// Attention over a sliding window of the paged cache for layers whose keys and values have different
// sizes and whose scores are more than a scaled dot product: a number per head multiplied into the score,
// the heads' scores mixed by a matrix before they become weights, a number per head added, and weights that
// are a softmax over the visible keys or a sigmoid of each score on its own (not normalised).
//
// The cache holds one row per token and key/value head: [key (dk) | value (dv)], pages of page_size tokens,
// so that a token's rows are the contiguous tail of its q/k/v product and are stored by one row copy.
//
//   cw_store_rows        copies columns [col0, col0 + width) of every token's row to the cache row its slot names
//   cw_window_attention  one flat batch of prompt portions and single tokens; a block per (token, part of its
//                        window); query head h reads key/value head h / (H / G); position p sees positions
//                        max(0, p - window + 1) .. p, all of which are in the cache when the kernel runs
//                        (`blocked`: positions are cut into blocks of `window` instead, and p sees the positions
//                        of its own block up to itself; `sink`: a logit per head that enters the softmax's
//                        denominator once, with no key and no value)
//   cw_rotate_store      turns the leading entries of every query and key head by the token's position (entry i with
//                        entry i + dims/2), writes the queries out and the rows [key | value] into the cache
//   cw_pool_rows         for every token that ends a block of `pool` positions: the mean of the block's rows [key | value]
//                        as the cache holds them, into the row of a second cache that the token's slot there names
//   (window_merge_kernel adds up the parts of a token's window; only launched when windows are cut)
// Further switches of cw_window_attention (WindowExtras; each usable alone): a window that never closes (window >= 2^30:
// plain causal attention); `pool`: beside the window, every block of `pool` positions that ends at or before p - window is
// seen as one key and value, read from the second cache (its rows come first in a row's order of keys); `softcap`: the
// score (after the numbers per head) becomes cap tanh(score / cap); `slopes`: slope[h] (p - j) is taken off the (capped)
// score; a query temperature: the score is multiplied by 1 + coef ln(floor((p + 1) / every) + 1) first of all; `gate`: head
// h's output is multiplied by sigmoid(gate[n, h]).
// bfloat16 calls run the tensor-core form further down when it takes the sizes; the CUDA-core kernel is the float32
// path and the fallback.
//
// Scores, weights, the softmax statistics and the weighted sums are float32 in both run precisions; T names
// the type of the product's output and of the cache.  A token's result depends on its position alone: keys
// are taken in tiles that start at the window's first position, in order, whatever else the step holds.
#include "common.cuh"

#define WA_MAX_COLS 16  // output columns per thread

template <typename T>
__global__ void __launch_bounds__(256)
store_rows_kernel(const T* __restrict__ src, int ld, int col0, int width, T* __restrict__ cache,
                  const int* __restrict__ slots, long long total_rows, int* __restrict__ status) {
    pdl_wait();
    const int n = blockIdx.x;
    const int slot = slots[n];
    if (slot < 0) return;  // padding of a fixed-shape step
    if (slot >= total_rows) {
        if (threadIdx.x == 0) cw_report(status, CW_ST_SLOT_RANGE, n, slot);
        return;
    }
    const T* from = src + (size_t)n * ld + col0;
    T* to = cache + (size_t)slot * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) to[c] = from[c];
}

extern "C" int cw_store_rows(const void* src, int ld, int col0, int width, void* cache, const int* slots, int N,
                             long long total_rows, int dtype, int* status, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || width <= 0 || col0 < 0 || ld < col0 + width || total_rows <= 0) return CW_ERR_BAD_SIZE;
    int threads = 32;
    while (threads < 256 && threads < width) threads *= 2;
    if (dtype == 0)
        return cw_launch_ordered(store_rows_kernel<float>, dim3(N), dim3(threads), 0, stream, (const float*)src, ld, col0, width,
                                 (float*)cache, slots, total_rows, status);
    if (dtype == 1)
        return cw_launch_ordered(store_rows_kernel<bf16>, dim3(N), dim3(threads), 0, stream, (const bf16*)src, ld, col0, width,
                                 (bf16*)cache, slots, total_rows, status);
    return CW_ERR_BAD_DTYPE;
}

// src [N, ld] float32: a token's product row [queries (H*dk) | per key/value head: key (dk), value (dv)].  The first
// `rot` entries of every query and key head are rotated: the pair (entry i, entry i + rot/2) by the angle
// position * inv_freq[i], in float32.  Queries go to q_out [N, H*dk], the rows [key | value] to the cache row that the
// token's slot names (slots null or < 0: nothing is stored).
template <typename T>
__global__ void __launch_bounds__(256)
rotate_store_kernel(const float* __restrict__ src, int ld, const int* __restrict__ positions, const int* __restrict__ tok_seq,
                    const int* __restrict__ slots, const float* __restrict__ inv_freq, int H, int G, int dk, int dv, int rot,
                    T* __restrict__ q_out, T* __restrict__ cache, long long total_rows, int* __restrict__ status) {
    pdl_wait();
    const int n = blockIdx.x;
    const int HQ = H * dk, row = dk + dv, half = rot >> 1;
    T* qo = q_out + (size_t)n * HQ;
    if (tok_seq[n] < 0) {  // padding of a fixed-shape step
        for (int c = threadIdx.x; c < HQ; c += blockDim.x) qo[c] = from_f<T>(0.f);
        return;
    }
    const float p = (float)positions[n];
    const float* x = src + (size_t)n * ld;
    auto turned = [&](const float* head, int i) {  // entry i (< rot) of a head after the rotation
        const int j = i < half ? i : i - half;
        float sn, cs;
        sincosf(p * inv_freq[j], &sn, &cs);
        return i < half ? head[i] * cs - head[i + half] * sn : head[i] * cs + head[i - half] * sn;
    };
    for (int c = threadIdx.x; c < HQ; c += blockDim.x) {
        const int h = c / dk, i = c - h * dk;
        qo[c] = from_f<T>(i < rot ? turned(x + (size_t)h * dk, i) : x[c]);
    }
    const int slot = slots != nullptr ? slots[n] : -1;
    if (slot < 0) return;
    if (slot >= total_rows) {
        if (threadIdx.x == 0) cw_report(status, CW_ST_SLOT_RANGE, n, slot);
        return;
    }
    T* to = cache + (size_t)slot * G * row;
    const float* kv = x + HQ;
    for (int c = threadIdx.x; c < G * row; c += blockDim.x) {
        const int g = c / row, i = c - g * row;
        to[c] = from_f<T>(i < rot ? turned(kv + (size_t)g * row, i) : kv[c]);
    }
}

extern "C" int cw_rotate_store(const float* src, int ld, const int* positions, const int* tok_seq, const int* slots,
                               const float* inv_freq, int N, int H, int G, int dk, int dv, int rot, void* q_out, void* cache,
                               long long total_rows, int dtype, int* status, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || rot < 0 || rot > dk || (rot & 1) || ld < H * dk + G * (dk + dv) ||
        (rot > 0 && inv_freq == nullptr) || total_rows < 0)
        return CW_ERR_BAD_SIZE;
    int threads = 64;
    while (threads < 256 && threads < H * dk) threads *= 2;
    if (dtype == 0)
        return cw_launch_ordered(rotate_store_kernel<float>, dim3(N), dim3(threads), 0, stream, src, ld, positions, tok_seq, slots, inv_freq,
                                 H, G, dk, dv, rot, (float*)q_out, (float*)cache, total_rows, status);
    if (dtype == 1)
        return cw_launch_ordered(rotate_store_kernel<bf16>, dim3(N), dim3(threads), 0, stream, src, ld, positions, tok_seq, slots, inv_freq,
                                 H, G, dk, dv, rot, (bf16*)q_out, (bf16*)cache, total_rows, status);
    return CW_ERR_BAD_DTYPE;
}

// ---- the means of whole blocks of positions -----------------------------------------------------------------
// A thread block per (token, 256 columns of its rows).  A token at position p with (p + 1) % pool == 0 ends the block of positions p - pool + 1 .. p: the
// mean of those positions' cache rows [G, dk + dv] (summed in float32 in the order of the positions, divided by pool, rounded
// once) goes to row pool_slots[n] of the second cache.  The positions' rows are in the cache when the kernel runs: the
// step's own tokens were stored before, and the cache manager keeps at least the last `pool` positions of a request.
template <typename T>
__global__ void __launch_bounds__(256)
pool_rows_kernel(const T* __restrict__ cache, const int* __restrict__ block_tables, int max_blocks, int page_size, int num_pages,
                 const int* __restrict__ positions, const int* __restrict__ tok_seq, const int* __restrict__ pool_slots,
                 T* __restrict__ pool_cache, long long pool_rows, int width, int pool, int* __restrict__ status) {
    pdl_wait();
    const int n = blockIdx.x;
    const int seq = tok_seq[n];
    if (seq < 0) return;
    const int p = positions[n];
    if ((p + 1) % pool != 0) return;
    const int slot = pool_slots[n];
    if (slot < 0) return;
    if (slot >= pool_rows) {
        if (threadIdx.x == 0) cw_report(status, CW_ST_SLOT_RANGE, n, slot);
        return;
    }
    __shared__ int rows[64];  // the cache rows of up to 64 positions of the block at a time (-1: none)
    const int* table = block_tables + (size_t)seq * max_blocks;
    const float inv = 1.0f / (float)pool;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    float sum = 0.f;
    for (int j0 = p - pool + 1; j0 <= p; j0 += 64) {
        const int count = min(64, p + 1 - j0);
        __syncthreads();  // the rows before are used up
        for (int i = threadIdx.x; i < count; i += blockDim.x) {
            const int j = j0 + i, blk = j / page_size;
            const int page = blk < max_blocks ? table[blk] : -1;
            if (page < 0 || page >= num_pages) {
                if (blockIdx.y == 0) cw_report(status, CW_ST_PAGE_RANGE, n, page);
                rows[i] = -1;
            } else {
                rows[i] = page * page_size + j % page_size;
            }
        }
        __syncthreads();
        if (c >= width) continue;
        // sixteen positions at a time: their loads are in flight together, the sum keeps the positions' order
        for (int i0 = 0; i0 < count; i0 += 16) {
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int row = i0 + i < count ? rows[i0 + i] : -1;
                v[i] = row >= 0 ? to_f(cache[(size_t)row * width + c]) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) sum += v[i];
        }
    }
    if (c < width) pool_cache[(size_t)slot * width + c] = from_f<T>(sum * inv);
}

extern "C" int cw_pool_rows(const void* cache, const int* block_tables, int max_blocks, int page_size, int num_pages,
                            const int* positions, const int* tok_seq, const int* pool_slots, void* pool_cache, long long pool_rows,
                            int width, int pool, int N, int dtype, int* status, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || width <= 0 || pool <= 0 || page_size <= 0 || max_blocks <= 0 || pool_rows <= 0) return CW_ERR_BAD_SIZE;
    int threads = 32;
    while (threads < 256 && threads < width) threads *= 2;
    const dim3 grid(N, (width + threads - 1) / threads);
    if (grid.y > 65535) return CW_ERR_UNSUPPORTED;
    if (dtype == 0)
        return cw_launch_ordered(pool_rows_kernel<float>, grid, dim3(threads), 0, stream, (const float*)cache, block_tables, max_blocks,
                                 page_size, num_pages, positions, tok_seq, pool_slots, (float*)pool_cache, pool_rows, width, pool, status);
    if (dtype == 1)
        return cw_launch_ordered(pool_rows_kernel<bf16>, grid, dim3(threads), 0, stream, (const bf16*)cache, block_tables, max_blocks,
                                 page_size, num_pages, positions, tok_seq, pool_slots, (bf16*)pool_cache, pool_rows, width, pool, status);
    return CW_ERR_BAD_DTYPE;
}

struct WindowAttentionArgs {
    const void* q;            // [N, ldq]: head h's query at columns h*dk ..
    int ldq;
    const void* cache;        // [rows, G, dk + dv]
    const int* block_tables;  // [S, max_blocks]
    int max_blocks, page_size, num_pages;
    const int* positions;     // [N]
    const int* tok_seq;       // [N], < 0: padding
    int H, G, dk, dv, window;
    float scale;
    const float* head_scale;  // [H] or null: multiplied into the score
    const float* talk;        // [H, H] or null: score_h <- sum_g talk[h, g] score_g
    const float* head_bias;   // [H] or null: added to the mixed score
    int sigmoid_weights;      // 0: softmax over the visible keys; 1: sigmoid of each score, not normalised
    int blocked;              // 0: p sees the last `window` positions; 1: p sees its own block of `window` positions up to itself
    const float* sink;        // [H] or null: a logit per head that counts once in the softmax's denominator
    void* out;                // [N, H*dv]
    int tile;                 // keys per tile (<= 32)
    int parts, part_keys;     // a token's window in `parts` pieces of `part_keys` keys (a multiple of tile)
    float* partial;           // parts > 1: [N, parts, H*dv + 2H] sums, running maxima and denominators
    int* status;
    // further switches (all off when zero or null)
    float softcap;            // > 0: score <- softcap tanh(score / softcap)
    const float* slopes;      // [H] or null: slopes[h] * (p - j) is taken off the score
    float temp_coef;          // with temp_every > 0: the score of a query at position p is multiplied by
    int temp_every;           //   1 + temp_coef ln(floor((p + 1) / temp_every) + 1)
    const float* gate;        // [N, ldg] or null: head h's output is multiplied by sigmoid(gate[n * ldg + h])
    int ldg;
    int pool;                 // > 0: blocks of `pool` positions that end at or before p - window are seen as one row each
    const void* pool_cache;   // [rows, G, dk + dv]: row b of a request is the mean of its positions b*pool .. b*pool + pool - 1
    const int* pool_tables;   // [S, pool_max_blocks]
    int pool_max_blocks, pool_pages;
};

// how many pooled blocks position p sees: those that end at or before p - window
__device__ __forceinline__ int wa_pooled_blocks(int p, int window, int pool) {
    const int behind = p - window + 1;  // positions before the window
    return pool > 0 && behind > 0 ? behind / pool : 0;
}
__device__ __forceinline__ float wa_query_temperature(int p, float coef, int every) {
    return every > 0 ? 1.f + coef * logf((float)((p + 1) / every + 1)) : 1.f;
}

template <typename T>
__global__ void __launch_bounds__(1024)
window_attention_kernel(const WindowAttentionArgs a) {
    extern __shared__ __align__(16) float wa_smem[];
    pdl_wait();
    const int n = blockIdx.x, part = blockIdx.y, tid = threadIdx.x;
    const int H = a.H, G = a.G, dk = a.dk, dv = a.dv, TK = a.tile;
    const int HV = H * dv, per = H / G, row_width = dk + dv;
    const int seq = a.tok_seq[n];
    T* out = (T*)a.out + (size_t)n * HV;
    float* partial = a.parts > 1 ? a.partial + ((size_t)n * a.parts + part) * (HV + 2 * H) : nullptr;
    if (seq < 0) {
        if (part == 0)
            for (int c = tid; c < HV; c += blockDim.x) out[c] = from_f<T>(0.f);
        return;
    }
    const int p = a.positions[n];
    const int first = a.blocked ? p - p % a.window : max(0, p - a.window + 1);
    // the row's keys in one order: its pooled blocks 0 .. nb-1, then the positions first .. p
    const int nb = wa_pooled_blocks(p, a.window, a.pool);
    const int lo = part * a.part_keys;
    const int total = nb + p + 1 - first;
    const int hi = part == a.parts - 1 ? total : min(total, lo + a.part_keys);  // keys lo .. hi-1 of that order (the last part: all the rest)
    const float temperature = wa_query_temperature(p, a.temp_coef, a.temp_every);
    const int GK = G * dk, kstride = GK | 1;
    float* qs = wa_smem;               // [H*dk]
    float* Ks = qs + H * dk;           // [TK][kstride]
    float* sc = Ks + TK * kstride;     // [H][TK] scaled dot products
    float* wt = sc + H * TK;           // [H][TK] weights
    float* mrun = wt + H * TK;         // [H] running maximum (softmax)
    float* lrun = mrun + H;            // [H] running denominator
    float* alpha = lrun + H;           // [H] what the sums so far are multiplied by when the maximum moves
    int* rows = (int*)(alpha + H);     // [TK] cache row of each key of the tile (-1: none)
    int* dist = rows + TK;             // [TK] how far back the key lies (p - j); -1: a pooled block (its row is in the second cache)
    const T* q = (const T*)a.q + (size_t)n * a.ldq;
    for (int i = tid; i < H * dk; i += blockDim.x) qs[i] = to_f(q[i]);
    for (int h = tid; h < H; h += blockDim.x) {
        mrun[h] = -INFINITY;
        lrun[h] = 0.f;
        alpha[h] = 1.f;
    }
    float acc[WA_MAX_COLS];
#pragma unroll
    for (int r = 0; r < WA_MAX_COLS; ++r) acc[r] = 0.f;
    const T* cache = (const T*)a.cache;
    const T* pool_cache = (const T*)a.pool_cache;
    const int* table = a.block_tables + (size_t)seq * a.max_blocks;
    const int* pool_table = a.pool > 0 ? a.pool_tables + (size_t)seq * a.pool_max_blocks : nullptr;
    const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
    for (int j0 = lo; j0 < hi; j0 += TK) {
        const int nk = min(TK, hi - j0);
        __syncthreads();  // the tile before is used up (and qs is written)
        if (tid < TK) {
            int row = -1, back = 0;
            if (tid < nk) {
                const int v = j0 + tid;
                if (v < nb) {  // a pooled block
                    const int blk = v / a.page_size;
                    const int page = blk < a.pool_max_blocks ? pool_table[blk] : -1;
                    if (page < 0 || page >= a.pool_pages)
                        cw_report(a.status, CW_ST_PAGE_RANGE, n, page);
                    else
                        row = page * a.page_size + v % a.page_size;
                    back = -1;
                } else {
                    const int pos = first + (v - nb), blk = pos / a.page_size;
                    const int page = blk < a.max_blocks ? table[blk] : -1;
                    if (page < 0 || page >= a.num_pages)
                        cw_report(a.status, CW_ST_PAGE_RANGE, n, page);
                    else
                        row = page * a.page_size + pos % a.page_size;
                    back = p - pos;
                }
            }
            rows[tid] = row;
            dist[tid] = back;
        }
        __syncthreads();
        for (int idx = tid; idx < nk * GK; idx += blockDim.x) {
            const int j = idx / GK, c = idx - j * GK;
            const int g = c / dk, i = c - g * dk;
            const int row = rows[j];
            const T* from = dist[j] < 0 ? pool_cache : cache;
            Ks[j * kstride + c] = row >= 0 ? to_f(from[((size_t)row * G + g) * row_width + i]) : 0.f;
        }
        __syncthreads();
        for (int pair = tid; pair < H * TK; pair += blockDim.x) {  // key fastest: rows of Ks an odd stride apart
            const int h = pair / TK, j = pair - h * TK;
            float dot = 0.f;
            if (j < nk) {
                const float* kr = Ks + j * kstride + (h / per) * dk;
                const float* qr = qs + h * dk;
                for (int i = 0; i < dk; ++i) dot = fmaf(qr[i], kr[i], dot);
            }
            sc[pair] = dot * a.scale * temperature;
        }
        __syncthreads();
        for (int h = warp; h < H; h += nwarps) {  // a warp per head, a lane per key of the tile
            float s = -INFINITY;
            const bool on = lane < nk && rows[lane] >= 0;
            if (on) {
                if (a.talk != nullptr) {
                    s = 0.f;
                    for (int g = 0; g < H; ++g) s = fmaf(a.talk[h * H + g], sc[g * TK + lane], s);
                } else {
                    s = sc[h * TK + lane];
                }
                if (a.head_scale != nullptr) s *= a.head_scale[h];
                if (a.head_bias != nullptr) s += a.head_bias[h];
                if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
                if (a.slopes != nullptr && dist[lane] > 0) s -= a.slopes[h] * (float)dist[lane];
            }
            if (a.sigmoid_weights) {
                if (lane < TK) wt[h * TK + lane] = on ? 1.f / (1.f + expf(-s)) : 0.f;
            } else {
                const float m_old = mrun[h];
                const float m_new = fmaxf(m_old, warp_max(s));
                const float e = on ? expf(s - m_new) : 0.f;
                const float sum = warp_sum(e);
                if (lane < TK) wt[h * TK + lane] = e;
                if (lane == 0) {
                    const float f = m_new == -INFINITY ? 1.f : expf(m_old - m_new);  // (exp(-inf) = 0 for the first tile)
                    alpha[h] = f;
                    lrun[h] = lrun[h] * f + sum;
                    mrun[h] = m_new;
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < WA_MAX_COLS; ++r) {
            const int col = tid + r * blockDim.x;
            if (col < HV) {
                const int h = col / dv, c = col - h * dv;
                const size_t voff = (size_t)(h / per) * row_width + dk + c;
                const float* w = wt + h * TK;
                float sum = a.sigmoid_weights ? acc[r] : acc[r] * alpha[h];
                for (int j = 0; j < nk; ++j) {
                    const int row = rows[j];
                    if (row >= 0) sum = fmaf(w[j], to_f((dist[j] < 0 ? pool_cache : cache)[(size_t)row * G * row_width + voff]), sum);
                }
                acc[r] = sum;
            }
        }
    }
    __syncthreads();
    if (a.sink != nullptr && partial == nullptr && !a.sigmoid_weights) {  // (cut windows: the merge adds it)
        for (int h = tid; h < H; h += blockDim.x)
            if (mrun[h] != -INFINITY) lrun[h] += expf(a.sink[h] - mrun[h]);
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < WA_MAX_COLS; ++r) {
        const int col = tid + r * blockDim.x;
        if (col < HV) {
            if (partial != nullptr) {
                partial[col] = acc[r];
            } else {
                const float l = a.sigmoid_weights ? 1.f : lrun[col / dv];
                float y = a.sigmoid_weights ? acc[r] : (l > 0.f ? acc[r] / l : 0.f);
                if (a.gate != nullptr) y *= 1.f / (1.f + expf(-a.gate[(size_t)n * a.ldg + col / dv]));
                out[col] = from_f<T>(y);
            }
        }
    }
    if (partial != nullptr)
        for (int h = tid; h < H; h += blockDim.x) {
            partial[HV + h] = mrun[h];
            partial[HV + H + h] = lrun[h];
        }
}

// The parts of a token's window, added up in part order: a block per (token, head), a thread per value column.
template <typename T>
__global__ void __launch_bounds__(256)
window_merge_kernel(const float* __restrict__ partial, const int* __restrict__ positions, const int* __restrict__ tok_seq,
                    int H, int dv, int window, int parts, int part_keys, int sigmoid_weights, int all_parts, int blocked,
                    const float* __restrict__ sink, T* __restrict__ out, int pool, const float* __restrict__ gate, int ldg) {
    __shared__ float factor[64];
    __shared__ float denominator;
    pdl_wait();
    const int n = blockIdx.x, h = blockIdx.y;
    if (tok_seq[n] < 0) return;  // (the attention kernel wrote the zeros)
    const int HV = H * dv, stride = HV + 2 * H;
    const int p = positions[n];
    const int keys = (blocked ? p % window + 1 : p + 1 - max(0, p - window + 1)) + wa_pooled_blocks(p, window, pool);
    const int used = all_parts ? parts : min(parts, (keys + part_keys - 1) / part_keys);  // (parts that hold none of the row's keys add nothing)
    const float* base = partial + (size_t)n * parts * stride;
    if (threadIdx.x == 0) {
        float m = -INFINITY, l = 0.f;
        if (!sigmoid_weights)
            for (int s = 0; s < used; ++s) m = fmaxf(m, base[(size_t)s * stride + HV + h]);
        for (int s = 0; s < used; ++s) {
            const float ms = base[(size_t)s * stride + HV + h];
            const float f = sigmoid_weights ? 1.f : (ms == -INFINITY ? 0.f : expf(ms - m));
            factor[s] = f;
            l = fmaf(f, base[(size_t)s * stride + HV + H + h], l);
        }
        if (sink != nullptr && !sigmoid_weights && m != -INFINITY) l += expf(sink[h] - m);
        denominator = sigmoid_weights ? 1.f : l;
    }
    __syncthreads();
    const float l = denominator;
    const float open = gate != nullptr ? 1.f / (1.f + expf(-gate[(size_t)n * ldg + h])) : 1.f;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        const int col = h * dv + c;
        float sum = 0.f;
        for (int s = 0; s < used; ++s) sum = fmaf(factor[s], base[(size_t)s * stride + col], sum);
        out[(size_t)n * HV + col] = from_f<T>((l > 0.f ? sum / l : 0.f) * open);
    }
}

// ---- the same on the tensor cores (bfloat16) -----------------------------------------------------------
// A block takes 16 consecutive query rows of one request and the query heads of GC key/value heads, a warp
// per query head (with `talk`, all heads: a weight needs every head's score of the same key).  Keys come in
// tiles of 32 through the block table into shared memory (cp.async, two stages when they fit); scores are
// mma.sync m16n8k16 products of bfloat16 queries and keys with float32 accumulators; scale, the heads' mix
// (through shared memory), the numbers per head, the window's mask and the weights (online softmax, or
// sigmoid) are float32 in registers; the weights go into the second product as two bfloat16 halves (hi + lo),
// so that they keep 16 bits of mantissa, against the values read with ldmatrix.trans as they lie in the cache.
// Blocks are mapped to (request, tile) by a scan of q_start, so a captured step needs nothing from the host.
#define WM_BN 32

struct WindowMmaArgs {
    WindowAttentionArgs w;
    const int* q_start;  // [S + 1]
    int S, N, gc, stages, all_parts;
};

__device__ __forceinline__ void wm_ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void wm_ldmatrix_x2(unsigned (&r)[2], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void wm_ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void wm_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void wm_cp16(void* smem, const void* gmem) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem) : "memory");
}
// two float32 weights as bfloat16 pairs: hi holds the rounded values, lo what the rounding left
__device__ __forceinline__ void wm_split(float x, float y, unsigned& hi, unsigned& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x - __low2float(h), y - __high2float(h));
    hi = *reinterpret_cast<const unsigned*>(&h);
    lo = *reinterpret_cast<const unsigned*>(&l);
}

template <int DVMAX>
__global__ void __launch_bounds__(DVMAX > 128 ? 256 : 512)
window_attention_mma_kernel(const WindowMmaArgs args) {
    extern __shared__ __align__(16) unsigned char wm_smem[];
    __shared__ int tile_seq, tile_row0, tile_rows;
    const WindowAttentionArgs& a = args.w;
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
    const int H = a.H, G = a.G, dk = a.dk, dv = a.dv, per = H / G, GC = args.gc;
    const int HV = H * dv, row_width = dk + dv;
    const int part = blockIdx.z;
    bf16* out = (bf16*)a.out;
    // rows of the flat batch that belong to no request (padding of a fixed-shape step) come out as zeros
    if (blockIdx.y == 0 && part == 0) {
        for (int i = 0; i < 16; ++i) {
            const int n = blockIdx.x * 16 + i;
            if (n < args.N && a.tok_seq[n] < 0)
                for (int c = tid; c < HV; c += blockDim.x) out[(size_t)n * HV + c] = from_f<bf16>(0.f);
        }
    }
    if (tid == 0) {  // which request and which 16 of its rows
        int b = blockIdx.x, seq = -1, row0 = 0, rows = 0;
        for (int s = 0; s < args.S; ++s) {
            const int st = args.q_start[s], len = args.q_start[s + 1] - st;
            if (len <= 0 || a.tok_seq[st] < 0) continue;
            const int t = (len + 15) >> 4;
            if (b < t) {
                seq = s;
                row0 = st + 16 * b;
                rows = min(16, st + len - row0);
                break;
            }
            b -= t;
        }
        tile_seq = seq;
        tile_row0 = row0;
        tile_rows = rows;
    }
    __syncthreads();
    const int seq = tile_seq, row0 = tile_row0, rows = tile_rows;
    if (seq < 0) return;
    const int g0 = blockIdx.y * GC;
    const int h = g0 * per + warp;  // this warp's query head
    const int gl = warp / per;      // its key/value head among the block's
    const int p0 = a.positions[row0];
    const int first = a.blocked ? p0 - p0 % a.window : max(0, p0 - a.window + 1);
    // What the tile's rows see, in key tiles of 32: the pooled blocks 0 .. NB-1 that its last row sees (tiles 0 .. pool_tiles-1,
    // the last of them part empty), then the positions first .. p0 + rows - 1; `parts` equal runs of whole key tiles.
    const int NB = wa_pooled_blocks(p0 + rows - 1, a.window, a.pool);
    const int pool_tiles = (NB + WM_BN - 1) / WM_BN;
    const int all_tiles = pool_tiles + (p0 + rows - first + WM_BN - 1) / WM_BN;
    const int part_tiles = (all_tiles + a.parts - 1) / a.parts;
    const int t_lo = part * part_tiles;
    const int t_hi = min(all_tiles, t_lo + part_tiles);  // key tiles t_lo .. t_hi-1
    const int hi = p0 + rows;                            // positions below hi
    // shared memory: Q [nwarps][16][dk+8], then per stage K [GC][32][dk+8] and V [GC][32][dv+8] (bfloat16), then with
    // talk the scores of all heads [H][16][40] and the mixing matrix [H][H] (float32)
    const int qs = dk + 8, ks_ = dk + 8, vs_ = dv + 8;
    bf16* Qs = (bf16*)wm_smem;
    bf16* KV = Qs + (size_t)nwarps * 16 * qs;
    const size_t stage_elems = (size_t)GC * WM_BN * (ks_ + vs_);
    float* Ss = (float*)(KV + (size_t)args.stages * stage_elems);
    float* Tm = Ss + (size_t)H * 16 * 40;
    const bool talk = a.talk != nullptr;
    const bf16* q = (const bf16*)a.q;
    for (int idx = tid; idx < nwarps * 16 * (dk / 8); idx += blockDim.x) {
        const int c = idx % (dk / 8), r = (idx / (dk / 8)) % 16, w = idx / (dk / 8) / 16;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *(const uint4*)(q + (size_t)(row0 + r) * a.ldq + (size_t)(g0 * per + w) * dk + c * 8);
        *(uint4*)(Qs + ((size_t)w * 16 + r) * qs + c * 8) = v;
    }
    if (talk)
        for (int i = tid; i < H * H; i += blockDim.x) Tm[i] = a.talk[i];
    const bf16* cache = (const bf16*)a.cache;
    const bf16* pool_cache = (const bf16*)a.pool_cache;
    const int* table = a.block_tables + (size_t)seq * a.max_blocks;
    const int* pool_table = a.pool > 0 ? a.pool_tables + (size_t)seq * a.pool_max_blocks : nullptr;
    // A thread copies the same 16-byte piece (key/value head g, piece c of the row) of every `kstep`-th key of a tile, so
    // that what does not change from tile to tile is worked out once; pages are found by a shift when their size is a
    // power of two.
    const int chunks_per_row = row_width / 8, kchunks = dk / 8;
    const int pieces = GC * chunks_per_row;                     // 16-byte pieces per key
    const bool strided = blockDim.x % pieces == 0 || pieces % blockDim.x == 0;
    const int page_shift = (a.page_size & (a.page_size - 1)) == 0 ? 31 - __clz(a.page_size) : -1;
    auto page_of = [&](int pos, int& offset) {
        int blk;
        if (page_shift >= 0) {
            blk = pos >> page_shift;
            offset = pos & (a.page_size - 1);
        } else {
            blk = pos / a.page_size;
            offset = pos - blk * a.page_size;
        }
        int page = blk < a.max_blocks ? table[blk] : -1;
        if (page < 0 || page >= a.num_pages) {
            cw_report(a.status, CW_ST_PAGE_RANGE, row0, page);
            page = -1;
        }
        return page;
    };
    auto pool_page_of = [&](int b, int& offset) {  // pooled block b of the request: its page in the second cache
        const int blk = b / a.page_size;
        offset = b - blk * a.page_size;
        int page = blk < a.pool_max_blocks ? pool_table[blk] : -1;
        if (page < 0 || page >= a.pool_pages) {
            cw_report(a.status, CW_ST_PAGE_RANGE, row0, page);
            page = -1;
        }
        return page;
    };
    auto copy_piece = [&](int j, int g, int c, int t, int stage) {  // key j of key tile t
        bf16* Kst = KV + (size_t)stage * stage_elems;
        bf16* Vst = Kst + (size_t)GC * WM_BN * ks_;
        bf16* dst = c < kchunks ? Kst + ((size_t)g * WM_BN + j) * ks_ + c * 8 : Vst + ((size_t)g * WM_BN + j) * vs_ + (c - kchunks) * 8;
        int offset = 0, page = -1;
        const bf16* from = cache;
        if (t < pool_tiles) {
            const int b = t * WM_BN + j;
            if (b < NB) page = pool_page_of(b, offset);
            from = pool_cache;
        } else {
            const int pos = first + (t - pool_tiles) * WM_BN + j;
            if (pos < hi) page = page_of(pos, offset);
        }
        if (page >= 0)
            wm_cp16(dst, from + (((size_t)page * a.page_size + offset) * G + g0 + g) * row_width + c * 8);
        else
            *(uint4*)dst = make_uint4(0, 0, 0, 0);
    };
    const int my_piece = tid % pieces, my_g = my_piece / chunks_per_row, my_c = my_piece - my_g * chunks_per_row;
    auto fetch = [&](int t, int stage) {  // the 32 keys of key tile t, of the block's key/value heads
        if (strided && blockDim.x >= pieces) {
            for (int j = tid / pieces; j < WM_BN; j += blockDim.x / pieces) copy_piece(j, my_g, my_c, t, stage);
        } else {
            for (int idx = tid; idx < WM_BN * pieces; idx += blockDim.x) {
                const int j = idx / pieces, piece = idx - j * pieces;
                const int g = piece / chunks_per_row;
                copy_piece(j, g, piece - g * chunks_per_row, t, stage);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float o[DVMAX / 8][4];
#pragma unroll
    for (int nt = 0; nt < DVMAX / 8; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int r_lo = lane >> 2, cpair = (lane & 3) * 2;  // this thread's rows r_lo and r_lo + 8, columns cpair, cpair + 1 of a tile of 8
    int row_first[2];  // the first position that each of the thread's two rows sees
    int row_blocks[2];  // how many pooled blocks it sees
    float row_temp[2];  // what its scores are multiplied by (a query temperature)
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int p = p0 + r_lo + 8 * x;
        row_first[x] = a.blocked ? p - p % a.window : p - a.window + 1;
        row_blocks[x] = wa_pooled_blocks(p, a.window, a.pool);
        row_temp[x] = wa_query_temperature(p, a.temp_coef, a.temp_every);
    }
    const bool bent = a.softcap > 0.f || a.slopes != nullptr || a.temp_every > 0;  // scores that are more than scaled and shifted
    const float slope = a.slopes != nullptr ? a.slopes[h] : 0.f;
    const int first_blocks = wa_pooled_blocks(p0, a.window, a.pool);  // pooled blocks that every row of the tile sees
    const int last_first = a.blocked ? (p0 + 15) - (p0 + 15) % a.window : p0 + 15 - a.window + 1;  // of the tile's last row
    const float head_scale = a.head_scale != nullptr ? a.head_scale[h] : 1.f;
    const float head_bias = a.head_bias != nullptr ? a.head_bias[h] : 0.f;
    const int nvt = dv / 8, nks = dk / 16;
    const int ntiles = t_hi > t_lo ? t_hi - t_lo : 0;
    if (ntiles > 0) fetch(t_lo, 0);
    for (int t = 0; t < ntiles; ++t) {
        const int kt = t_lo + t;              // the key tile
        const bool pooled = kt < pool_tiles;  // its keys are pooled blocks kt*32 .., else positions j0 ..
        const int j0 = pooled ? kt * WM_BN : first + (kt - pool_tiles) * WM_BN;
        const int stage = args.stages == 2 ? (t & 1) : 0;
        if (args.stages == 2 && t + 1 < ntiles) {
            fetch(kt + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            if (args.stages == 1 && t > 0) fetch(kt, 0);  // one stage: everyone left it at the end of the last round
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // the tile has landed (and Q, at the first)
        const bf16* Kt = KV + (size_t)stage * stage_elems + (size_t)gl * WM_BN * ks_;
        const bf16* Vt = KV + (size_t)stage * stage_elems + (size_t)GC * WM_BN * ks_ + (size_t)gl * WM_BN * vs_;
        float s[WM_BN / 8][4];
#pragma unroll
        for (int nt = 0; nt < WM_BN / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        for (int ks = 0; ks < nks; ++ks) {
            unsigned qa[4];
            wm_ldmatrix_x4(qa, Qs + ((size_t)warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * qs + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nt = 0; nt < WM_BN / 8; nt += 2) {  // sixteen keys at a time: lanes 0-15 address the first eight, 16-31 the next
                unsigned kb[4];
                wm_ldmatrix_x4(kb, Kt + (size_t)(nt * 8 + (lane & 7) + (lane >> 4) * 8) * ks_ + ks * 16 + ((lane >> 3) & 1) * 8);
                wm_mma(s[nt], qa, kb[0], kb[1]);
                wm_mma(s[nt + 1], qa, kb[2], kb[3]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < WM_BN / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] *= a.scale;
        if (talk) {  // every head's scores of this tile through shared memory, then this head's mix of them
#pragma unroll
            for (int nt = 0; nt < WM_BN / 8; ++nt) {
                *(float2*)(Ss + ((size_t)h * 16 + r_lo) * 40 + nt * 8 + cpair) = make_float2(s[nt][0], s[nt][1]);
                *(float2*)(Ss + ((size_t)h * 16 + r_lo + 8) * 40 + nt * 8 + cpair) = make_float2(s[nt][2], s[nt][3]);
            }
            __syncthreads();
#pragma unroll
            for (int nt = 0; nt < WM_BN / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
            for (int g = 0; g < H; ++g) {
                const float w = Tm[h * H + g];
#pragma unroll
                for (int nt = 0; nt < WM_BN / 8; ++nt) {
                    const float2 u = *(const float2*)(Ss + ((size_t)g * 16 + r_lo) * 40 + nt * 8 + cpair);
                    const float2 v = *(const float2*)(Ss + ((size_t)g * 16 + r_lo + 8) * 40 + nt * 8 + cpair);
                    s[nt][0] = fmaf(w, u.x, s[nt][0]);
                    s[nt][1] = fmaf(w, u.y, s[nt][1]);
                    s[nt][2] = fmaf(w, v.x, s[nt][2]);
                    s[nt][3] = fmaf(w, v.y, s[nt][3]);
                }
            }
        }
        // the window's mask and the weights
        float tile_max[2] = {-INFINITY, -INFINITY};
        // (a tile that every row sees whole needs no mask: its last key is not behind the first row, its first not
        // before the last row's window)
        const bool whole = pooled ? rows == 16 && j0 + WM_BN <= first_blocks
                                  : rows == 16 && j0 + WM_BN - 1 <= p0 && j0 >= last_first && j0 + WM_BN <= hi;
#pragma unroll
        for (int nt = 0; nt < WM_BN / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                bool on = true;
                const int j = j0 + nt * 8 + cpair + (e & 1);
                if (!whole) {
                    const int row = r_lo + (e >> 1) * 8;
                    const int p = p0 + row;
                    on = pooled ? row < rows && j < row_blocks[e >> 1] : row < rows && j <= p && j >= row_first[e >> 1] && j < hi;
                }
                float v = s[nt][e];
                if (bent) v *= row_temp[e >> 1];
                v = fmaf(v, head_scale, head_bias);
                if (bent) {
                    if (a.softcap > 0.f) v = a.softcap * tanhf(v / a.softcap);
                    if (!pooled) v -= slope * (float)(p0 + r_lo + (e >> 1) * 8 - j);
                }
                v = on ? v : -INFINITY;
                s[nt][e] = v;
                tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
            }
        if (a.sigmoid_weights) {
#pragma unroll
            for (int nt = 0; nt < WM_BN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = s[nt][e] == -INFINITY ? 0.f : 1.f / (1.f + __expf(-s[nt][e]));
        } else {
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                float tm = tile_max[x];
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
                const float m_new = fmaxf(m_run[x], tm);
                const float f = m_new == -INFINITY ? 1.f : __expf(m_run[x] - m_new);
                float sum = 0.f;
#pragma unroll
                for (int nt = 0; nt < WM_BN / 8; ++nt)
#pragma unroll
                    for (int e = 2 * x; e < 2 * x + 2; ++e) {
                        const float w = s[nt][e] == -INFINITY ? 0.f : __expf(s[nt][e] - m_new);
                        s[nt][e] = w;
                        sum += w;
                    }
                l_run[x] = fmaf(l_run[x], f, sum);
                m_run[x] = m_new;
#pragma unroll
                for (int nt = 0; nt < DVMAX / 8; ++nt) {
                    o[nt][2 * x] *= f;
                    o[nt][2 * x + 1] *= f;
                }
            }
        }
        unsigned a_hi[2][4], a_lo[2][4];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            wm_split(s[2 * kk][0], s[2 * kk][1], a_hi[kk][0], a_lo[kk][0]);
            wm_split(s[2 * kk][2], s[2 * kk][3], a_hi[kk][1], a_lo[kk][1]);
            wm_split(s[2 * kk + 1][0], s[2 * kk + 1][1], a_hi[kk][2], a_lo[kk][2]);
            wm_split(s[2 * kk + 1][2], s[2 * kk + 1][3], a_hi[kk][3], a_lo[kk][3]);
        }
        // four tiles of value columns at a time, so that consecutive products go to different accumulators
#pragma unroll
        for (int nb = 0; nb < DVMAX / 8; nb += 4) {
            if (nb < nvt) {
                unsigned vb[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (nb + i < nvt) wm_ldmatrix_x4_trans(vb[i], Vt + (size_t)lane * vs_ + (nb + i) * 8);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (nb + i < nvt) wm_mma(o[nb + i], a_hi[0], vb[i][0], vb[i][1]);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (nb + i < nvt) wm_mma(o[nb + i], a_lo[0], vb[i][0], vb[i][1]);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (nb + i < nvt) wm_mma(o[nb + i], a_hi[1], vb[i][2], vb[i][3]);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (nb + i < nvt) wm_mma(o[nb + i], a_lo[1], vb[i][2], vb[i][3]);
            }
        }
        __syncthreads();  // everyone is done with this stage (and with the shared scores)
    }
    // results: rows r_lo and r_lo + 8 of this warp's head
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        l_run[x] += __shfl_xor_sync(0xffffffffu, l_run[x], 1);
        l_run[x] += __shfl_xor_sync(0xffffffffu, l_run[x], 2);
        if (a.sink != nullptr && a.parts == 1 && !a.sigmoid_weights && m_run[x] != -INFINITY)  // (cut rows: the merge adds it)
            l_run[x] += __expf(a.sink[h] - m_run[x]);
    }
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int row = r_lo + 8 * x;
        if (row >= rows) continue;
        const size_t n = (size_t)row0 + row;
        if (a.parts > 1) {
            float* pr = a.partial + (n * a.parts + part) * (HV + 2 * H);
#pragma unroll
            for (int nt = 0; nt < DVMAX / 8; ++nt)
                if (nt < nvt) *(float2*)(pr + (size_t)h * dv + nt * 8 + cpair) = make_float2(o[nt][2 * x], o[nt][2 * x + 1]);
            if ((lane & 3) == 0) {
                pr[HV + h] = m_run[x];
                pr[HV + H + h] = l_run[x];
            }
        } else {
            float inv = a.sigmoid_weights ? 1.f : (l_run[x] > 0.f ? 1.f / l_run[x] : 0.f);
            if (a.gate != nullptr) inv *= 1.f / (1.f + __expf(-a.gate[n * a.ldg + h]));
#pragma unroll
            for (int nt = 0; nt < DVMAX / 8; ++nt)
                if (nt < nvt)
                    *(__nv_bfloat162*)(out + n * HV + (size_t)h * dv + nt * 8 + cpair) = __floats2bfloat162_rn(o[nt][2 * x] * inv, o[nt][2 * x + 1] * inv);
        }
    }
}

static int g_window_mma = 1;
extern "C" int cw_window_attention_set_mma(int on) { g_window_mma = on ? 1 : 0; return CW_OK; }

// The tensor-core form if it takes the sizes (returns 1 and launches), else 0; negative or positive: an error.
static int window_attention_mma(const WindowAttentionArgs& base, const int* q_start, int S, int N, cudaStream_t stream, int* launched) {
    *launched = 0;
    const int H = base.H, G = base.G, dk = base.dk, dv = base.dv, per = H / G;
    if (!g_window_mma || q_start == nullptr || dk % 16 || dv % 8 || dv > 256 || per > 16 || base.ldq % 8 || ((uintptr_t)base.q & 15) ||
        ((uintptr_t)base.cache & 15))
        return 0;
    const int max_warps = dv > 128 ? 8 : 16;
    int gc;
    if (base.talk != nullptr) {
        gc = G;
    } else {
        gc = per >= 4 ? 1 : min(G, 4 / per);
        while (G % gc) --gc;
    }
    const int nwarps = gc * per;
    if (nwarps > max_warps) return 0;
    auto bytes = [&](int stages) {
        return sizeof(bf16) * ((size_t)nwarps * 16 * (dk + 8) + (size_t)stages * gc * WM_BN * (dk + dv + 16)) +
               (base.talk != nullptr ? sizeof(float) * ((size_t)H * 16 * 40 + (size_t)H * H) : 0);
    };
    int stages = 2;
    if (bytes(2) > (200u << 10)) stages = 1;
    const size_t smem = bytes(stages);
    if (smem > (200u << 10)) return 0;
    WindowMmaArgs args = {base, q_start, S, N, gc, stages, 1};
    const int which = dv <= 64 ? 0 : (dv <= 128 ? 1 : 2);
    using Kernel = void (*)(const WindowMmaArgs);
    const Kernel kernels[3] = {window_attention_mma_kernel<64>, window_attention_mma_kernel<128>, window_attention_mma_kernel<256>};
    static size_t allowed[3] = {48 << 10, 48 << 10, 48 << 10};
    if (smem > allowed[which]) {
        const cudaError_t e = cudaFuncSetAttribute(kernels[which], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed[which] = smem;
    }
    *launched = 1;
    const dim3 grid((N + 15) / 16 + S, G / gc, base.parts);
    return cw_launch_ordered(kernels[which], grid, dim3(nwarps * 32), smem, stream, args);
}

// How many floats of `partial` a call with these sizes needs (0: windows are not cut).
extern "C" long long cw_window_attention_partial_words(int N, int H, int dv, int parts) {
    return parts > 1 ? (long long)N * parts * (H * dv + 2 * H) : 0;
}

extern "C" int cw_window_attention(const void* q, int ldq, const void* cache, const int* block_tables, int max_blocks,
                                   int page_size, int num_pages, const int* positions, const int* tok_seq, int N, int H,
                                   int G, int dk, int dv, int window, float scale, const float* head_scale,
                                   const float* talk, const float* head_bias, int sigmoid_weights, int blocked, const float* sink,
                                   void* out, int parts, float* partial, const int* q_start, int S, int dtype, int* status,
                                   float softcap, const float* slopes, float temp_coef, int temp_every, const float* gate, int ldg,
                                   int pool, const void* pool_cache, const int* pool_tables, int pool_max_blocks, int pool_pages,
                                   cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (softcap < 0.f || temp_every < 0 || pool < 0 || (gate != nullptr && ldg < H)) return CW_ERR_BAD_SIZE;
    if (pool > 0 && (pool_cache == nullptr || pool_tables == nullptr || pool_max_blocks <= 0 || pool_pages <= 0 || blocked || slopes != nullptr))
        return CW_ERR_BAD_SIZE;  // (a pooled block has no distance, and blocks of positions have nothing before them)
    if (N < 0 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || window <= 0 || page_size <= 0 || max_blocks <= 0 ||
        ldq < H * dk || parts < 1)
        return CW_ERR_BAD_SIZE;
    if (parts > 1 && partial == nullptr) return CW_ERR_BAD_SIZE;
    const int HV = H * dv;
    if (parts > 64) return CW_ERR_BAD_SIZE;
    int merge_threads = 32;
    while (merge_threads < 256 && merge_threads < dv) merge_threads *= 2;
    if (dtype == 1) {  // bfloat16: the tensor-core form when it takes the sizes
        const WindowAttentionArgs base = {q, ldq, cache, block_tables, max_blocks, page_size, num_pages, positions, tok_seq, H, G, dk, dv,
                                          window, scale, head_scale, talk, head_bias, sigmoid_weights, blocked, sink, out, WM_BN, parts, 0,
                                          partial, status, softcap, slopes, temp_coef, temp_every, gate, ldg, pool, pool_cache, pool_tables,
                                          pool_max_blocks, pool_pages};
        int launched = 0;
        const int rc = window_attention_mma(base, q_start, S, N, stream, &launched);
        if (rc != 0) return rc;
        if (launched) {
            if (parts == 1) return CW_OK;
            return cw_launch_ordered(window_merge_kernel<bf16>, dim3(N, H), dim3(merge_threads), 0, stream, (const float*)partial, positions, tok_seq, H,
                                     dv, window, parts, 0, sigmoid_weights, 1, blocked, sink, (bf16*)out, pool, gate, ldg);
        }
    }
    int threads = 128;
    while (threads < 1024 && threads * 4 < HV) threads *= 2;      // about four output columns a thread
    while (threads * WA_MAX_COLS < HV && threads < 1024) threads *= 2;
    if (threads * WA_MAX_COLS < HV) return CW_ERR_UNSUPPORTED;
    // keys per tile: as many (up to 32) as leave the staged keys within 64 KB
    const int kstride = (G * dk) | 1;
    int tile = 32;
    while (tile > 4 && (size_t)tile * kstride * sizeof(float) > (64u << 10)) tile >>= 1;
    const size_t smem = sizeof(float) * ((size_t)H * dk + (size_t)tile * kstride + 2 * (size_t)H * tile + 3 * (size_t)H) +
                        sizeof(int) * 2 * tile;
    if (smem > (200u << 10)) return CW_ERR_UNSUPPORTED;
    // (a row's order of keys is cut in `parts` runs: float32 runs never cut, so the longest row that a cut must cover is a
    // window and the pooled blocks before it; a window that never closes is cut as if it held 2^20 keys)
    const long long longest = (long long)min(window, 1 << 20) + (pool > 0 ? (1 << 20) / pool : 0);
    int part_keys = (int)((longest + parts - 1) / parts);
    part_keys = (part_keys + tile - 1) / tile * tile;
    WindowAttentionArgs a = {q, ldq, cache, block_tables, max_blocks, page_size, num_pages, positions, tok_seq, H, G, dk, dv,
                             window, scale, head_scale, talk, head_bias, sigmoid_weights, blocked, sink, out, tile, parts, part_keys,
                             partial, status, softcap, slopes, temp_coef, temp_every, gate, ldg, pool, pool_cache, pool_tables,
                             pool_max_blocks, pool_pages};
    static size_t allowed[2] = {48 << 10, 48 << 10};
    if (dtype != 0 && dtype != 1) return CW_ERR_BAD_DTYPE;
    if (smem > allowed[dtype]) {
        const cudaError_t e = dtype == 0
            ? cudaFuncSetAttribute(window_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
            : cudaFuncSetAttribute(window_attention_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed[dtype] = smem;
    }
    const dim3 grid(N, parts);
    int rc = dtype == 0 ? cw_launch_ordered(window_attention_kernel<float>, grid, dim3(threads), smem, stream, a)
                        : cw_launch_ordered(window_attention_kernel<bf16>, grid, dim3(threads), smem, stream, a);
    if (rc != 0 || parts == 1) return rc;
    if (dtype == 0)
        return cw_launch_ordered(window_merge_kernel<float>, dim3(N, H), dim3(merge_threads), 0, stream, (const float*)partial, positions, tok_seq,
                                 H, dv, window, parts, part_keys, sigmoid_weights, 0, blocked, sink, (float*)out, pool, gate, ldg);
    return cw_launch_ordered(window_merge_kernel<bf16>, dim3(N, H), dim3(merge_threads), 0, stream, (const float*)partial, positions, tok_seq, H,
                             dv, window, parts, part_keys, sigmoid_weights, 0, blocked, sink, (bf16*)out, pool, gate, ldg);
}

CW_TRACE_TU(window_attention)
