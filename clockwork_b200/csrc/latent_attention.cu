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
        return cw_launch_ordered(latent_prepare_kernel<float>, dim3(N), dim3(128), 0, stream, down, (const float*)q, (float*)qa,
                         (float*)cache, norm_w, inv_freq, positions, slots, H, dim, rot, rank, num_slots, eps, write_cache, status);
    if (dtype == 1)
        return cw_launch_ordered(latent_prepare_kernel<bf16>, dim3(N), dim3(128), 0, stream, down, (const bf16*)q, (bf16*)qa,
                         (bf16*)cache, norm_w, inv_freq, positions, slots, H, dim, rot, rank, num_slots, eps, write_cache, status);
    return CW_ERR_BAD_DTYPE;
}

// One block per (token, group of LA_HB heads).  Keys in chunks of 128, a thread per key for the scores
// (all LA_HB heads at once, so a cached row is read once per group), then a thread per latent column for
// the weighted sum.  The chunking depends on the token's position only, never on the rest of the batch.
#define LA_CH 128
#define LA_HB 4
#define LA_NC 8  // latent columns per thread: rank <= LA_CH * LA_NC

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

// ---- the same on the tensor cores (bfloat16 cache and queries) -------------------------------------------
// One block per (token, group of 16 heads): the 16 heads are the rows of an mma.sync m16n8k16 tile, so a
// cached row is read once for all of them.  Keys in tiles of 64 (cp.async through the block table, rows
// past the token's position filled with zeros).  Warp w computes the scores of keys 16w..16w+15 over the
// whole row width; maxima and sums meet in shared memory (added in warp order); the weights go to shared
// memory as two bfloat16 halves (p = hi + lo, so the product with the latents carries float32 weights to
// 16 bits of mantissa); every warp then owns a quarter of the latent's columns and accumulates them over
// all 64 keys, the cached tile itself being the second operand (read transposed by ldmatrix).
#define LT_KEYS 64
#define LT_NT 16   // n-tiles of 8 latent columns per warp: rank <= 4 * 8 * LT_NT
#define LT_PLD 72  // row of the weights in shared memory, in elements

__device__ __forceinline__ void lt_cp16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void lt_ldm(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lt_ldm_t(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lt_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned lt_pack(bf16 a, bf16 b) {
    return (unsigned)__bfloat16_as_ushort(a) | ((unsigned)__bfloat16_as_ushort(b) << 16);
}

__global__ void __launch_bounds__(128)
latent_attention_mma_kernel(const bf16* __restrict__ qa, bf16* __restrict__ out, const bf16* __restrict__ cache,
                            const int* __restrict__ block_tables, const int* __restrict__ tok_seq,
                            const int* __restrict__ positions, const float* __restrict__ sink, int H, int rank, int rot,
                            int page_size, int max_blocks, int num_pages, float scale, int* status) {
    extern __shared__ __align__(16) unsigned char lt_smem[];
    const int D = rank + rot, LDK = D + 8;
    bf16* Ks = (bf16*)lt_smem;                 // [LT_KEYS][LDK]
    bf16* Qs = Ks + (size_t)LT_KEYS * LDK;     // [16][LDK]
    bf16* Phi = Qs + (size_t)16 * LDK;         // [16][LT_PLD]
    bf16* Plo = Phi + 16 * LT_PLD;
    float* row_max = (float*)(Plo + 16 * LT_PLD);  // [4][16]
    float* row_sum = row_max + 64;                  // [4][16]
    int* slot_s = (int*)(row_sum + 64);             // [LT_KEYS]
    pdl_wait();
    const int t = blockIdx.x, h0 = blockIdx.y * 16, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int heads = min(16, H - h0);
    const int seq = tok_seq[t];
    if (seq < 0) {  // padding row of a fixed-shape batch
        for (int i = tid; i < heads * rank; i += 128) out[((size_t)t * H + h0) * rank + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int chunks = D / 8;  // 16-byte pieces of a row
    for (int idx = tid; idx < 16 * chunks; idx += 128) {
        const int r = idx / chunks, c = idx - r * chunks;
        lt_cp16(Qs + (size_t)r * LDK + c * 8, qa + ((size_t)t * H + h0 + (r < heads ? r : 0)) * D + c * 8, r < heads);
    }
    const int kv_end = positions[t] + 1;
    const int* table = block_tables + (size_t)seq * max_blocks;
    const int ntiles = rank / 8;                       // n-tiles of the latent
    const int per_warp = (ntiles + 3) / 4;
    const int first_nt = warp * per_warp;
    const int my_nt = max(0, min(per_warp, ntiles - first_nt));
    const int g = lane >> 2, q4 = lane & 3;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows g and g + 8
    float acc[LT_NT][4];
#pragma unroll
    for (int i = 0; i < LT_NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    for (int k0 = 0; k0 < kv_end; k0 += LT_KEYS) {
        if (tid < LT_KEYS) {
            const int j = k0 + tid;
            int slot = -1;
            if (j < kv_end) {
                const int blk = j / page_size;
                const int page = blk < max_blocks ? table[blk] : -1;
                if (page < 0 || page >= num_pages)
                    cw_report(status, CW_ST_PAGE_RANGE, t, page);
                else
                    slot = page * page_size + j % page_size;
            }
            slot_s[tid] = slot;
        }
        __syncthreads();  // (also: everyone has left the tile before)
        for (int idx = tid; idx < LT_KEYS * chunks; idx += 128) {
            const int r = idx / chunks, c = idx - r * chunks;
            const int slot = slot_s[r];
            lt_cp16(Ks + (size_t)r * LDK + c * 8, cache + (size_t)(slot < 0 ? 0 : slot) * D + c * 8, slot >= 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // scores of this warp's 16 keys
        float s[2][4] = {};
        for (int kk = 0; kk < D; kk += 16) {
            unsigned a[4], b[4];
            lt_ldm(a, Qs + (size_t)(lane & 15) * LDK + kk + (lane >> 4) * 8);
            lt_ldm(b, Ks + (size_t)(warp * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + kk + ((lane >> 3) & 1) * 8);
            lt_mma(s[0], a, b[0], b[1]);
            lt_mma(s[1], a, b[2], b[3]);
        }
        float top0 = -INFINITY, top1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = k0 + warp * 16 + nt * 8 + q4 * 2 + (e & 1);
                s[nt][e] = key < kv_end && slot_s[key - k0] >= 0 ? s[nt][e] * scale : -INFINITY;
                if (e < 2) top0 = fmaxf(top0, s[nt][e]); else top1 = fmaxf(top1, s[nt][e]);
            }
        top0 = fmaxf(top0, __shfl_xor_sync(0xffffffffu, top0, 1));
        top0 = fmaxf(top0, __shfl_xor_sync(0xffffffffu, top0, 2));
        top1 = fmaxf(top1, __shfl_xor_sync(0xffffffffu, top1, 1));
        top1 = fmaxf(top1, __shfl_xor_sync(0xffffffffu, top1, 2));
        if (q4 == 0) {
            row_max[warp * 16 + g] = top0;
            row_max[warp * 16 + g + 8] = top1;
        }
        __syncthreads();
        float n0 = m0, n1 = m1;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            n0 = fmaxf(n0, row_max[w * 16 + g]);
            n1 = fmaxf(n1, row_max[w * 16 + g + 8]);
        }
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) p[e] = s[nt][e] == -INFINITY ? 0.f : expf(s[nt][e] - (e < 2 ? n0 : n1));
            sum0 += p[0] + p[1];
            sum1 += p[2] + p[3];
            bf16 hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                hi[e] = __float2bfloat16_rn(p[e]);
                lo[e] = __float2bfloat16_rn(p[e] - __bfloat162float(hi[e]));
            }
            const int col = warp * 16 + nt * 8 + q4 * 2;
            *(unsigned*)(Phi + g * LT_PLD + col) = lt_pack(hi[0], hi[1]);
            *(unsigned*)(Phi + (g + 8) * LT_PLD + col) = lt_pack(hi[2], hi[3]);
            *(unsigned*)(Plo + g * LT_PLD + col) = lt_pack(lo[0], lo[1]);
            *(unsigned*)(Plo + (g + 8) * LT_PLD + col) = lt_pack(lo[2], lo[3]);
        }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        if (q4 == 0) {
            row_sum[warp * 16 + g] = sum0;
            row_sum[warp * 16 + g + 8] = sum1;
        }
        __syncthreads();
        const float alpha0 = m0 == -INFINITY ? 0.f : expf(m0 - n0), alpha1 = m1 == -INFINITY ? 0.f : expf(m1 - n1);
        float t0 = 0.f, t1 = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {  // in warp order: the same sum in every thread
            t0 += row_sum[w * 16 + g];
            t1 += row_sum[w * 16 + g + 8];
        }
        l0 = l0 * alpha0 + t0;
        l1 = l1 * alpha1 + t1;
        m0 = n0;
        m1 = n1;
#pragma unroll
        for (int i = 0; i < LT_NT; ++i) {
            acc[i][0] *= alpha0;
            acc[i][1] *= alpha0;
            acc[i][2] *= alpha1;
            acc[i][3] *= alpha1;
        }
        // weights (16 x 64) times this warp's columns of the cached tile (64 x 8 my_nt)
#pragma unroll
        for (int ks = 0; ks < LT_KEYS / 16; ++ks) {
            unsigned ah[4], al[4];
            lt_ldm(ah, Phi + (lane & 15) * LT_PLD + ks * 16 + (lane >> 4) * 8);
            lt_ldm(al, Plo + (lane & 15) * LT_PLD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < LT_NT / 2; ++np) {
                if (np * 2 < my_nt) {
                    unsigned b[4];
                    lt_ldm_t(b, Ks + (size_t)(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (first_nt + np * 2) * 8 + (lane >> 4) * 8);
                    lt_mma(acc[np * 2], ah, b[0], b[1]);
                    lt_mma(acc[np * 2], al, b[0], b[1]);
                    lt_mma(acc[np * 2 + 1], ah, b[2], b[3]);  // (an odd count's last pair also fills a tile that is not stored)
                    lt_mma(acc[np * 2 + 1], al, b[2], b[3]);
                }
            }
        }
    }
    // the sink joins the denominator only
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = g + half * 8;
        if (r >= heads) continue;
        const float m = half ? m1 : m0, l = half ? l1 : l0;
        const float sk = sink != nullptr ? sink[h0 + r] : -INFINITY;
        const float top = fmaxf(m, sk);
        const float keep = m == -INFINITY ? 0.f : expf(m - top);
        const float denom = l * keep + (sk == -INFINITY ? 0.f : expf(sk - top));
        const float inv = denom > 0.f ? keep / denom : 0.f;
        bf16* o = out + ((size_t)t * H + h0 + r) * rank;
#pragma unroll
        for (int i = 0; i < LT_NT; ++i) {
            if (i < my_nt) {
                const int col = (first_nt + i) * 8 + q4 * 2;
                *(unsigned*)(o + col) = lt_pack(__float2bfloat16_rn(acc[i][half * 2] * inv), __float2bfloat16_rn(acc[i][half * 2 + 1] * inv));
            }
        }
    }
}

static int g_latent_mma = 1;
extern "C" int cw_latent_attention_set_mma(int on) { g_latent_mma = on ? 1 : 0; return CW_OK; }

extern "C" int cw_latent_attention(const void* qa, void* out, const void* cache, const int* block_tables, const int* tok_seq,
                                   const int* positions, const float* sink, int N, int H, int rank, int rot, int page_size,
                                   int max_blocks, int num_pages, float scale, int dtype, int* status, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || H <= 0 || rank <= 0 || rot < 0 || page_size <= 0 || max_blocks <= 0) return CW_ERR_BAD_SIZE;
    if (rank > LA_CH * LA_NC || (H + LA_HB - 1) / LA_HB > 65535) return CW_ERR_UNSUPPORTED;
    const size_t smem = (size_t)LA_HB * (rank + rot) * sizeof(float);
    dim3 grid(N, (H + LA_HB - 1) / LA_HB);
    if (dtype == 0)
        return cw_launch_ordered(latent_attention_kernel<float, float>, grid, dim3(LA_CH), smem, stream, (const float*)qa, (float*)out,
                         (const float*)cache, block_tables, tok_seq, positions, sink, H, rank, rot, page_size, max_blocks,
                         num_pages, scale, status);
    const int D = rank + rot;
    if (dtype == 1 && g_latent_mma && D % 16 == 0 && rank % 8 == 0 && rank <= 4 * 8 * LT_NT && (H + 15) / 16 <= 65535 &&
        ((uintptr_t)qa & 15) == 0 && ((uintptr_t)cache & 15) == 0 && ((uintptr_t)out & 3) == 0) {
        const size_t bytes = (size_t)(LT_KEYS + 16) * (D + 8) * sizeof(bf16) + 2 * 16 * LT_PLD * sizeof(bf16) + 128 * sizeof(float) +
                             LT_KEYS * sizeof(int);
        static size_t allowed = 48 << 10;
        if (bytes > allowed) {
            const cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            if (e != cudaSuccess) return (int)e;
            allowed = bytes;
        }
        return cw_launch_ordered(latent_attention_mma_kernel, dim3(N, (H + 15) / 16), dim3(128), bytes, stream, (const bf16*)qa, (bf16*)out,
                         (const bf16*)cache, block_tables, tok_seq, positions, sink, H, rank, rot, page_size, max_blocks, num_pages,
                         scale, status);
    }
    if (dtype == 1)
        return cw_launch_ordered(latent_attention_kernel<bf16, bf16>, grid, dim3(LA_CH), smem, stream, (const bf16*)qa, (bf16*)out,
                         (const bf16*)cache, block_tables, tok_seq, positions, sink, H, rank, rot, page_size, max_blocks,
                         num_pages, scale, status);
    return CW_ERR_BAD_DTYPE;
}

CW_TRACE_TU(latent_attention)
