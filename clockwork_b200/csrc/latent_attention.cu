// Attention over a cached latent: per token the cache keeps one row [c | k_r] (a normed latent of
// `rank` numbers and one rotated key part of `rot` numbers shared by all heads) instead of keys and
// values per head.  The per-head products are moved to the query side: with q_h = [q_plain | q_rot],
//
//   score_h(j) = (q_plain . (W_uk,h c_j) + q_rot . k_r,j) scale = ((W_uk,h^T q_plain) . c_j + q_rot . k_r,j) scale
//   out_h      = W_uv,h (sum_j p_h(j) c_j),   p_h(j) = exp(s_j) / (exp(sink_h) + sum_j' exp(s_j'))
//
// so a query row is [W_uk,h^T q_plain | q_rot] (rank + rot numbers per head, made by a grouped product
// and cw_latent_prepare), all heads read the same cached rows, and the kernel returns sum_j p c_j per
// head for another grouped product to map to the head's value size.  The sink is a learned number per
// head that takes part in the softmax denominator only (no key, no value, not scaled, counted once).
//
//   cw_latent_prepare    RMS norm of the latent (float32) and rotation of the shared key part, written to
//                        the cache row of the token's slot; rotation of the queries' rotated parts
//   cw_latent_attention  causal attention of a flat batch (prompt portions beside single tokens) over the
//                        paged rows; float32 scores, weights and accumulation in both run precisions
#include "common.cuh"

// down [N, rank + rot] float32 (the projection's output), q [N, H*(dim+rot)], qa [N, H*(rank+rot)] (the
// rotated parts are written at [.., rank:]), cache [slots, rank + rot].  Pair (i, i + rot/2) at position p
// turns by the angle p * inv_freq[i].
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const float* __restrict__ down, const T* __restrict__ q, T* __restrict__ qa, T* __restrict__ cache,
                      const float* __restrict__ norm_w, const float* __restrict__ inv_freq,
                      const int* __restrict__ positions, const int* __restrict__ slots, int H, int dim, int rot, int rank,
                      int num_slots, float eps, int write_cache, int* status) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const int D = rank + rot, half = rot / 2;
    const float pos = (float)positions[row];
    const float* dr = down + (size_t)row * D;
    int slot = write_cache ? slots[row] : -1;
    if (slot >= num_slots) {
        if (tid == 0) cw_report(status, CW_ST_SLOT_RANGE, row, slot);
        slot = -1;
    }
    float ss = 0.f;
    for (int i = tid; i < rank; i += blockDim.x) ss = fmaf(dr[i], dr[i], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    if (slot >= 0) {
        T* cr = cache + (size_t)slot * D;
        for (int i = tid; i < rank; i += blockDim.x) cr[i] = from_f<T>(dr[i] * inv * norm_w[i]);
        for (int i = tid; i < half; i += blockDim.x) {
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            const float u = dr[rank + i], v = dr[rank + half + i];
            cr[rank + i] = from_f<T>(u * cs - v * sn);
            cr[rank + half + i] = from_f<T>(v * cs + u * sn);
        }
    }
    for (int idx = tid; idx < H * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        const T* qr = q + (size_t)row * H * (dim + rot) + (size_t)h * (dim + rot) + dim;
        const float u = to_f(qr[i]), v = to_f(qr[half + i]);
        T* o = qa + (size_t)row * H * D + (size_t)h * D + rank;
        o[i] = from_f<T>(u * cs - v * sn);
        o[half + i] = from_f<T>(v * cs + u * sn);
    }
}

extern "C" int cw_latent_prepare(const float* down, const void* q, void* qa, void* cache, const float* norm_w,
                                 const float* inv_freq, const int* positions, const int* slots, int N, int H, int dim, int rot,
                                 int rank, int num_slots, float eps, int write_cache, int dtype, int* status,
                                 cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || H <= 0 || dim < 0 || rot < 0 || rot % 2 || rank <= 0) return CW_ERR_BAD_SIZE;
    if (dtype == 0)
        return cw_launch(latent_prepare_kernel<float>, dim3(N), dim3(128), 0, stream, 1, down, (const float*)q, (float*)qa,
                         (float*)cache, norm_w, inv_freq, positions, slots, H, dim, rot, rank, num_slots, eps, write_cache, status);
    if (dtype == 1)
        return cw_launch(latent_prepare_kernel<bf16>, dim3(N), dim3(128), 0, stream, 1, down, (const bf16*)q, (bf16*)qa,
                         (bf16*)cache, norm_w, inv_freq, positions, slots, H, dim, rot, rank, num_slots, eps, write_cache, status);
    return CW_ERR_BAD_DTYPE;
}

// One block per (token, group of LA_HB heads).  Keys in chunks of 128, a thread per key for the scores
// (all LA_HB heads at once, so a cached row is read once per group), then a thread per latent column for
// the weighted sum.  The chunking depends on the token's position only, never on the rest of the batch.
#define LA_CH 128
#define LA_HB 4
#define LA_NC 4  // latent columns per thread: rank <= LA_CH * LA_NC

// max or sum of LA_HB values per thread over the block, in a fixed order
template <bool MAX>
__device__ __forceinline__ void block_reduce_heads(float (&v)[LA_HB], float (*buf)[LA_HB]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int h = 0; h < LA_HB; ++h) v[h] = MAX ? warp_max(v[h]) : warp_sum(v[h]);
    __syncthreads();
    if (lane == 0)
        for (int h = 0; h < LA_HB; ++h) buf[warp][h] = v[h];
    __syncthreads();
#pragma unroll
    for (int h = 0; h < LA_HB; ++h) {
        float r = buf[0][h];
        for (int w = 1; w < LA_CH / 32; ++w) r = MAX ? fmaxf(r, buf[w][h]) : r + buf[w][h];
        v[h] = r;
    }
}

template <typename T, typename TO>
__global__ void __launch_bounds__(LA_CH)
latent_attention_kernel(const T* __restrict__ qa, TO* __restrict__ out, const T* __restrict__ cache,
                        const int* __restrict__ block_tables, const int* __restrict__ tok_seq,
                        const int* __restrict__ positions, const float* __restrict__ sink, int H, int rank, int rot,
                        int page_size, int max_blocks, int num_pages, float scale, int* status) {
    extern __shared__ float q_s[];  // [LA_HB][D]
    __shared__ float p_s[LA_HB][LA_CH];
    __shared__ int slot_s[LA_CH];
    __shared__ float red_s[LA_CH / 32][LA_HB];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h0 = blockIdx.y * LA_HB, tid = threadIdx.x;
    const int D = rank + rot;
    const int seq = tok_seq[t];
    const int heads = min(LA_HB, H - h0);
    if (seq < 0) {  // padding row of a fixed-shape batch
        for (int i = tid; i < heads * rank; i += LA_CH) out[((size_t)t * H + h0) * rank + i] = from_f<TO>(0.f);
        return;
    }
    for (int i = tid; i < LA_HB * D; i += LA_CH) {
        const int hb = i / D, d = i % D;
        q_s[i] = hb < heads ? to_f(qa[((size_t)t * H + h0 + hb) * D + d]) : 0.f;
    }
    __syncthreads();
    const int kv_end = positions[t] + 1;
    const int* table = block_tables + (size_t)seq * max_blocks;
    float m[LA_HB], l[LA_HB], acc[LA_HB][LA_NC];
#pragma unroll
    for (int hb = 0; hb < LA_HB; ++hb) {
        m[hb] = -INFINITY;
        l[hb] = 0.f;
#pragma unroll
        for (int c = 0; c < LA_NC; ++c) acc[hb][c] = 0.f;
    }
    for (int c0 = 0; c0 < kv_end; c0 += LA_CH) {
        const int j = c0 + tid;
        float s[LA_HB];
#pragma unroll
        for (int hb = 0; hb < LA_HB; ++hb) s[hb] = -INFINITY;
        int slot = -1;
        if (j < kv_end) {
            const int blk = j / page_size;
            const int page = blk < max_blocks ? table[blk] : -1;
            if (page < 0 || page >= num_pages) {
                cw_report(status, CW_ST_PAGE_RANGE, t, page);
            } else {
                slot = page * page_size + j % page_size;
                const T* kp = cache + (size_t)slot * D;
                float dot[LA_HB] = {};
                for (int d = 0; d < D; ++d) {
                    const float kd = to_f(kp[d]);
#pragma unroll
                    for (int hb = 0; hb < LA_HB; ++hb) dot[hb] = fmaf(q_s[hb * D + d], kd, dot[hb]);
                }
#pragma unroll
                for (int hb = 0; hb < LA_HB; ++hb) s[hb] = dot[hb] * scale;
            }
        }
        slot_s[tid] = slot;
        float top[LA_HB];
#pragma unroll
        for (int hb = 0; hb < LA_HB; ++hb) top[hb] = s[hb];
        block_reduce_heads<true>(top, red_s);
        float p[LA_HB], alpha[LA_HB];
#pragma unroll
        for (int hb = 0; hb < LA_HB; ++hb) {
            const float m_new = fmaxf(m[hb], top[hb]);
            p[hb] = slot >= 0 ? expf(s[hb] - m_new) : 0.f;
            p_s[hb][tid] = p[hb];
            alpha[hb] = m[hb] == -INFINITY ? 0.f : expf(m[hb] - m_new);
            m[hb] = m_new;
        }
        block_reduce_heads<false>(p, red_s);  // (its barriers also order p_s and slot_s before the reads below)
#pragma unroll
        for (int hb = 0; hb < LA_HB; ++hb) {
            l[hb] = l[hb] * alpha[hb] + p[hb];
#pragma unroll
            for (int c = 0; c < LA_NC; ++c) acc[hb][c] *= alpha[hb];
        }
        const int n = min(LA_CH, kv_end - c0);
        for (int jj = 0; jj < n; ++jj) {
            const int sl = slot_s[jj];
            if (sl < 0) continue;
            const T* cp = cache + (size_t)sl * D;
#pragma unroll
            for (int c = 0; c < LA_NC; ++c) {
                const int col = tid + c * LA_CH;
                if (col < rank) {
                    const float cv = to_f(cp[col]);
#pragma unroll
                    for (int hb = 0; hb < LA_HB; ++hb) acc[hb][c] = fmaf(p_s[hb][jj], cv, acc[hb][c]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int hb = 0; hb < LA_HB; ++hb) {
        if (hb >= heads) continue;
        const float sk = sink != nullptr ? sink[h0 + hb] : -INFINITY;
        const float top = fmaxf(m[hb], sk);
        const float keep = m[hb] == -INFINITY ? 0.f : expf(m[hb] - top);
        const float denom = l[hb] * keep + (sk == -INFINITY ? 0.f : expf(sk - top));
        const float inv = denom > 0.f ? keep / denom : 0.f;
#pragma unroll
        for (int c = 0; c < LA_NC; ++c) {
            const int col = tid + c * LA_CH;
            if (col < rank) out[((size_t)t * H + h0 + hb) * rank + col] = from_f<TO>(acc[hb][c] * inv);
        }
    }
}

extern "C" int cw_latent_attention(const void* qa, void* out, const void* cache, const int* block_tables, const int* tok_seq,
                                   const int* positions, const float* sink, int N, int H, int rank, int rot, int page_size,
                                   int max_blocks, int num_pages, float scale, int dtype, int* status, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || H <= 0 || rank <= 0 || rot < 0 || page_size <= 0 || max_blocks <= 0) return CW_ERR_BAD_SIZE;
    if (rank > LA_CH * LA_NC || (H + LA_HB - 1) / LA_HB > 65535) return CW_ERR_UNSUPPORTED;
    const size_t smem = (size_t)LA_HB * (rank + rot) * sizeof(float);
    dim3 grid(N, (H + LA_HB - 1) / LA_HB);
    if (dtype == 0)
        return cw_launch(latent_attention_kernel<float, float>, grid, dim3(LA_CH), smem, stream, 1, (const float*)qa, (float*)out,
                         (const float*)cache, block_tables, tok_seq, positions, sink, H, rank, rot, page_size, max_blocks,
                         num_pages, scale, status);
    if (dtype == 1)
        return cw_launch(latent_attention_kernel<bf16, bf16>, grid, dim3(LA_CH), smem, stream, 1, (const bf16*)qa, (bf16*)out,
                         (const bf16*)cache, block_tables, tok_seq, positions, sink, H, rank, rot, page_size, max_blocks,
                         num_pages, scale, status);
    return CW_ERR_BAD_DTYPE;
}

CW_TRACE_TU(latent_attention)
