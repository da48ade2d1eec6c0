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
//   cw_window_merge      adds up the parts of a token's window (only launched when windows are cut)
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
    void* out;                // [N, H*dv]
    int tile;                 // keys per tile (<= 32)
    int parts, part_keys;     // a token's window in `parts` pieces of `part_keys` keys (a multiple of tile)
    float* partial;           // parts > 1: [N, parts, H*dv + 2H] sums, running maxima and denominators
    int* status;
};

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
    const int first = max(0, p - a.window + 1);
    const int lo = first + part * a.part_keys;
    const int hi = min(p + 1, lo + a.part_keys);  // keys lo .. hi-1
    const int GK = G * dk, kstride = GK | 1;
    float* qs = wa_smem;               // [H*dk]
    float* Ks = qs + H * dk;           // [TK][kstride]
    float* sc = Ks + TK * kstride;     // [H][TK] scaled dot products
    float* wt = sc + H * TK;           // [H][TK] weights
    float* mrun = wt + H * TK;         // [H] running maximum (softmax)
    float* lrun = mrun + H;            // [H] running denominator
    float* alpha = lrun + H;           // [H] what the sums so far are multiplied by when the maximum moves
    int* rows = (int*)(alpha + H);     // [TK] cache row of each key of the tile (-1: none)
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
    const int* table = a.block_tables + (size_t)seq * a.max_blocks;
    const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
    for (int j0 = lo; j0 < hi; j0 += TK) {
        const int nk = min(TK, hi - j0);
        __syncthreads();  // the tile before is used up (and qs is written)
        if (tid < TK) {
            int row = -1;
            if (tid < nk) {
                const int pos = j0 + tid, blk = pos / a.page_size;
                const int page = blk < a.max_blocks ? table[blk] : -1;
                if (page < 0 || page >= a.num_pages)
                    cw_report(a.status, CW_ST_PAGE_RANGE, n, page);
                else
                    row = page * a.page_size + pos % a.page_size;
            }
            rows[tid] = row;
        }
        __syncthreads();
        for (int idx = tid; idx < nk * GK; idx += blockDim.x) {
            const int j = idx / GK, c = idx - j * GK;
            const int g = c / dk, i = c - g * dk;
            const int row = rows[j];
            Ks[j * kstride + c] = row >= 0 ? to_f(cache[((size_t)row * G + g) * row_width + i]) : 0.f;
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
            sc[pair] = dot * a.scale;
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
                const T* vcol = cache + (size_t)(h / per) * row_width + dk + c;
                const float* w = wt + h * TK;
                float sum = a.sigmoid_weights ? acc[r] : acc[r] * alpha[h];
                for (int j = 0; j < nk; ++j) {
                    const int row = rows[j];
                    if (row >= 0) sum = fmaf(w[j], to_f(vcol[(size_t)row * G * row_width]), sum);
                }
                acc[r] = sum;
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < WA_MAX_COLS; ++r) {
        const int col = tid + r * blockDim.x;
        if (col < HV) {
            if (partial != nullptr) {
                partial[col] = acc[r];
            } else {
                const float l = a.sigmoid_weights ? 1.f : lrun[col / dv];
                out[col] = from_f<T>(a.sigmoid_weights ? acc[r] : (l > 0.f ? acc[r] / l : 0.f));
            }
        }
    }
    if (partial != nullptr)
        for (int h = tid; h < H; h += blockDim.x) {
            partial[HV + h] = mrun[h];
            partial[HV + H + h] = lrun[h];
        }
}

// The parts of a token's window, added up in part order.
template <typename T>
__global__ void __launch_bounds__(256)
window_merge_kernel(const float* __restrict__ partial, const int* __restrict__ positions, const int* __restrict__ tok_seq,
                    int H, int dv, int window, int parts, int part_keys, int sigmoid_weights, T* __restrict__ out) {
    pdl_wait();
    const int n = blockIdx.x;
    if (tok_seq[n] < 0) return;  // (the attention kernel wrote the zeros)
    const int HV = H * dv, stride = HV + 2 * H;
    const int p = positions[n];
    const int keys = p + 1 - max(0, p - window + 1);
    const int used = (keys + part_keys - 1) / part_keys;
    const float* base = partial + (size_t)n * parts * stride;
    for (int col = threadIdx.x; col < HV; col += blockDim.x) {
        const int h = col / dv;
        float sum = 0.f, l = 0.f;
        if (sigmoid_weights) {
            for (int s = 0; s < used; ++s) sum += base[(size_t)s * stride + col];
            l = 1.f;
        } else {
            float m = -INFINITY;
            for (int s = 0; s < used; ++s) m = fmaxf(m, base[(size_t)s * stride + HV + h]);
            for (int s = 0; s < used; ++s) {
                const float ms = base[(size_t)s * stride + HV + h];
                const float f = ms == -INFINITY ? 0.f : expf(ms - m);
                sum = fmaf(f, base[(size_t)s * stride + col], sum);
                l = fmaf(f, base[(size_t)s * stride + HV + H + h], l);
            }
        }
        out[(size_t)n * HV + col] = from_f<T>(l > 0.f ? sum / l : 0.f);
    }
}

// How many floats of `partial` a call with these sizes needs (0: windows are not cut).
extern "C" long long cw_window_attention_partial_words(int N, int H, int dv, int parts) {
    return parts > 1 ? (long long)N * parts * (H * dv + 2 * H) : 0;
}

extern "C" int cw_window_attention(const void* q, int ldq, const void* cache, const int* block_tables, int max_blocks,
                                   int page_size, int num_pages, const int* positions, const int* tok_seq, int N, int H,
                                   int G, int dk, int dv, int window, float scale, const float* head_scale,
                                   const float* talk, const float* head_bias, int sigmoid_weights, void* out, int parts,
                                   float* partial, int dtype, int* status, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || window <= 0 || page_size <= 0 || max_blocks <= 0 ||
        ldq < H * dk || parts < 1)
        return CW_ERR_BAD_SIZE;
    if (parts > 1 && partial == nullptr) return CW_ERR_BAD_SIZE;
    const int HV = H * dv;
    int threads = 128;
    while (threads < 1024 && threads * 4 < HV) threads *= 2;      // about four output columns a thread
    while (threads * WA_MAX_COLS < HV && threads < 1024) threads *= 2;
    if (threads * WA_MAX_COLS < HV) return CW_ERR_UNSUPPORTED;
    // keys per tile: as many (up to 32) as leave the staged keys within 64 KB
    const int kstride = (G * dk) | 1;
    int tile = 32;
    while (tile > 4 && (size_t)tile * kstride * sizeof(float) > (64u << 10)) tile >>= 1;
    const size_t smem = sizeof(float) * ((size_t)H * dk + (size_t)tile * kstride + 2 * (size_t)H * tile + 3 * (size_t)H) +
                        sizeof(int) * tile;
    if (smem > (200u << 10)) return CW_ERR_UNSUPPORTED;
    int part_keys = (window + parts - 1) / parts;
    part_keys = (part_keys + tile - 1) / tile * tile;
    WindowAttentionArgs a = {q, ldq, cache, block_tables, max_blocks, page_size, num_pages, positions, tok_seq, H, G, dk, dv,
                             window, scale, head_scale, talk, head_bias, sigmoid_weights, out, tile, parts, part_keys, partial,
                             status};
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
        return cw_launch_ordered(window_merge_kernel<float>, dim3(N), dim3(256), 0, stream, (const float*)partial, positions, tok_seq,
                                 H, dv, window, parts, part_keys, sigmoid_weights, (float*)out);
    return cw_launch_ordered(window_merge_kernel<bf16>, dim3(N), dim3(256), 0, stream, (const float*)partial, positions, tok_seq, H,
                             dv, window, parts, part_keys, sigmoid_weights, (bf16*)out);
}

CW_TRACE_TU(window_attention)
