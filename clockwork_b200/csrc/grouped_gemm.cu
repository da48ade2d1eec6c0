// Matrix products in groups: every group g has its own weight matrix B_g [Nout, K] and its own rows
// of A.  Two callers: a mixture of experts (group = expert, its rows are the (token, choice) pairs
// routed to it, gathered through an index) and per-head products of an attention layer that keeps a
// latent instead of keys (group = head, every token is a row, A and C are column slices per head).
//
//   C[dst(r), c_group_off*g + n] = epilogue( sum_k A[src(r), a_group_off*g + k] * B_g[n, k] )
//
// float32 accumulation in k order on the CUDA cores in both run precisions: a row's result depends on
// the row and its group only, never on which other rows share its tile.
//
// Beside it the router of a mixture of experts (float32 logits, the `top` largest, softmax over the
// chosen), the grouping of (token, choice) pairs by expert, and the weighted sum of the experts'
// outputs into the float32 residual, in choice order.
#include "common.cuh"

#define GG_TM 32
#define GG_TN 64
#define GG_TK 32

#define GG_EPI_STORE 0        // C (T) = acc
#define GG_EPI_STORE_F32 1    // C (float) = acc
#define GG_EPI_SILU_MUL 2     // C (T) = silu(acc) * acc2, acc2 from B2
#define GG_EPI_SIGMOID_GATE 3 // C (T) = acc * sigmoid(gate[dst, c_group_off*g + n])

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const T* __restrict__ A, int lda, int a_group_off, const T* __restrict__ B, const T* __restrict__ B2,
                    long long b_stride, void* __restrict__ Cv, int ldc, int c_group_off,
                    const int* __restrict__ offsets, const int* __restrict__ a_index, int a_div,
                    const int* __restrict__ c_index, const T* __restrict__ gate, int ldg,
                    int M, int Nout, int K, int G) {
    __shared__ float As[GG_TK][GG_TM + 1];
    __shared__ float Bs[GG_TK][GG_TN + 1];
    __shared__ float B2s[EPI == GG_EPI_SILU_MUL ? GG_TK : 1][GG_TN + 1];
    __shared__ int src_s[GG_TM], dst_s[GG_TM];
    pdl_launch_dependents();
    pdl_wait();
    // which group and which tile of its rows
    int g, row0, rows_end;
    if (offsets == nullptr) {
        const int tiles = (M + GG_TM - 1) / GG_TM;
        g = blockIdx.x / tiles;
        row0 = (blockIdx.x % tiles) * GG_TM;
        rows_end = M;
    } else {
        int tile = blockIdx.x;
        g = 0;
        while (g < G) {
            const int n = offsets[g + 1] - offsets[g];
            const int t = (n + GG_TM - 1) / GG_TM;
            if (tile < t) break;
            tile -= t;
            ++g;
        }
        if (g >= G) return;
        row0 = offsets[g] + tile * GG_TM;
        rows_end = offsets[g + 1];
    }
    const int tid = threadIdx.x;
    if (tid < GG_TM) {
        const int r = row0 + tid;
        int s = -1, d = -1;
        if (r < rows_end) {
            s = a_index != nullptr ? a_index[r] / a_div : r;
            d = c_index != nullptr ? c_index[r] : r;
        }
        src_s[tid] = s;
        dst_s[tid] = d;
    }
    __syncthreads();
    const int n0 = blockIdx.y * GG_TN;
    const T* Bg = B + (size_t)g * b_stride;
    const T* B2g = EPI == GG_EPI_SILU_MUL ? B2 + (size_t)g * b_stride : nullptr;
    const int tx = tid & 15, ty = tid >> 4;  // 4 columns x 2 rows per thread
    float acc[2][4] = {}, acc2[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += GG_TK) {
        for (int idx = tid; idx < GG_TM * GG_TK; idx += 256) {
            const int r = idx / GG_TK, kk = idx % GG_TK;
            const int s = src_s[r];
            As[kk][r] = (s >= 0 && k0 + kk < K) ? to_f(A[(size_t)s * lda + (size_t)g * a_group_off + k0 + kk]) : 0.f;
        }
        for (int idx = tid; idx < GG_TN * GG_TK; idx += 256) {
            const int n = idx / GG_TK, kk = idx % GG_TK;
            const bool on = n0 + n < Nout && k0 + kk < K;
            Bs[kk][n] = on ? to_f(Bg[(size_t)(n0 + n) * K + k0 + kk]) : 0.f;
            if (EPI == GG_EPI_SILU_MUL) B2s[kk][n] = on ? to_f(B2g[(size_t)(n0 + n) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < GG_TK; ++kk) {
            const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float b = Bs[kk][tx * 4 + c];
                acc[0][c] = fmaf(a0, b, acc[0][c]);
                acc[1][c] = fmaf(a1, b, acc[1][c]);
                if (EPI == GG_EPI_SILU_MUL) {
                    const float b2 = B2s[kk][tx * 4 + c];
                    acc2[0][c] = fmaf(a0, b2, acc2[0][c]);
                    acc2[1][c] = fmaf(a1, b2, acc2[1][c]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int d = dst_s[ty * 2 + r];
        if (d < 0) continue;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int n = n0 + tx * 4 + c;
            if (n >= Nout) continue;
            const size_t at = (size_t)d * ldc + (size_t)g * c_group_off + n;
            float v = acc[r][c];
            if (EPI == GG_EPI_STORE_F32) {
                ((float*)Cv)[at] = v;
            } else {
                if (EPI == GG_EPI_SILU_MUL) v = v / (1.f + expf(-v)) * acc2[r][c];
                if (EPI == GG_EPI_SIGMOID_GATE) v = v / (1.f + expf(-to_f(gate[(size_t)d * ldg + (size_t)g * c_group_off + n])));
                ((T*)Cv)[at] = from_f<T>(v);
            }
        }
    }
}

template <typename T>
static int launch_grouped(int epi, dim3 grid, cudaStream_t stream, const void* A, int lda, int a_group_off, const void* B,
                          const void* B2, long long b_stride, void* C, int ldc, int c_group_off, const int* offsets,
                          const int* a_index, int a_div, const int* c_index, const void* gate, int ldg, int M, int Nout, int K,
                          int G) {
#define GG_GO(E)                                                                                                              \
    return cw_launch(grouped_gemm_kernel<T, E>, grid, dim3(256), 0, stream, 1, (const T*)A, lda, a_group_off, (const T*)B,    \
                     (const T*)B2, b_stride, C, ldc, c_group_off, offsets, a_index, a_div, c_index, (const T*)gate, ldg, M,   \
                     Nout, K, G)
    switch (epi) {
        case GG_EPI_STORE: GG_GO(GG_EPI_STORE);
        case GG_EPI_STORE_F32: GG_GO(GG_EPI_STORE_F32);
        case GG_EPI_SILU_MUL: GG_GO(GG_EPI_SILU_MUL);
        case GG_EPI_SIGMOID_GATE: GG_GO(GG_EPI_SIGMOID_GATE);
    }
#undef GG_GO
    return CW_ERR_UNSUPPORTED;
}

// offsets == null: every group has the M rows 0..M-1.  Otherwise group g owns the sorted rows
// offsets[g]..offsets[g+1]-1 (at most M in all), row r reads A row a_index[r] / a_div and writes C row
// c_index[r] (identity where the index is null).
extern "C" int cw_grouped_gemm(const void* A, int lda, int a_group_off, const void* B, const void* B2, long long b_stride,
                               void* C, int ldc, int c_group_off, const int* offsets, const int* a_index, int a_div,
                               const int* c_index, const void* gate, int ldg, int M, int Nout, int K, int G, int epilogue,
                               int dtype, cudaStream_t stream) {
    if (M == 0) return CW_OK;
    if (M < 0 || Nout <= 0 || K <= 0 || G <= 0 || a_div <= 0) return CW_ERR_BAD_SIZE;
    if (epilogue == GG_EPI_SILU_MUL && B2 == nullptr) return CW_ERR_BAD_SIZE;
    if (epilogue == GG_EPI_SIGMOID_GATE && gate == nullptr) return CW_ERR_BAD_SIZE;
    const long long tiles = offsets == nullptr ? (long long)G * ((M + GG_TM - 1) / GG_TM) : (long long)(M + GG_TM - 1) / GG_TM + G;
    if (tiles > 0x7fffffffLL) return CW_ERR_UNSUPPORTED;
    dim3 grid((unsigned)tiles, (Nout + GG_TN - 1) / GG_TN);
    if (dtype == 0)
        return launch_grouped<float>(epilogue, grid, stream, A, lda, a_group_off, B, B2, b_stride, C, ldc, c_group_off, offsets,
                                     a_index, a_div, c_index, gate, ldg, M, Nout, K, G);
    if (dtype == 1)
        return launch_grouped<bf16>(epilogue, grid, stream, A, lda, a_group_off, B, B2, b_stride, C, ldc, c_group_off, offsets,
                                    a_index, a_div, c_index, gate, ldg, M, Nout, K, G);
    return CW_ERR_BAD_DTYPE;
}

// ---- router ---------------------------------------------------------------------------------------
// logits = Wr x + b in float32 (x as the run stores it); the `top` largest (the lower index wins a
// tie); weights = softmax over the chosen logits.  sel < 0 marks a padding row.
template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ x, const float* __restrict__ Wr, const float* __restrict__ b,
                  const int* __restrict__ tok_seq, int* __restrict__ sel, float* __restrict__ wt, int W, int E, int top) {
    extern __shared__ float logit_s[];  // [E] logits, then [top] chosen logits
    float* chosen_s = logit_s + E;
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (tok_seq[row] < 0) {
        for (int t = threadIdx.x; t < top; t += blockDim.x) {
            sel[(size_t)row * top + t] = -1;
            wt[(size_t)row * top + t] = 0.f;
        }
        return;
    }
    const T* xr = x + (size_t)row * W;
    for (int e = warp; e < E; e += 4) {
        const float* w = Wr + (size_t)e * W;
        float acc = 0.f;
        for (int c = lane; c < W; c += 32) acc = fmaf(to_f(xr[c]), w[c], acc);
        acc = warp_sum(acc);
        if (lane == 0) logit_s[e] = acc + (b != nullptr ? b[e] : 0.f);
    }
    __syncthreads();
    if (warp != 0) return;
    for (int t = 0; t < top; ++t) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = logit_s[e];
            if (v > best) best = v, at = e;  // ascending e: the first of equals stays
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ov > best || (ov == best && oa < at)) best = ov, at = oa;
        }
        if (at == 0x7fffffff) at = t % E;  // no finite logit left (never with finite inputs)
        if (lane == 0) {
            sel[(size_t)row * top + t] = at;
            chosen_s[t] = best;
            logit_s[at] = -INFINITY;
        }
        __syncwarp();
    }
    const float first = chosen_s[0];
    float total = 0.f;
    for (int t = 0; t < top; ++t) total += expf(chosen_s[t] - first);  // the same order in every lane
    for (int t = lane; t < top; t += 32) wt[(size_t)row * top + t] = expf(chosen_s[t] - first) / total;
}

extern "C" int cw_moe_route(const void* x, const float* Wr, const float* b, const int* tok_seq, int* sel, float* wt, int N,
                            int W, int E, int top, int dtype, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || W <= 0 || E <= 0 || top <= 0 || top > E) return CW_ERR_BAD_SIZE;
    if (E + top > 8192) return CW_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(E + top) * sizeof(float);
    if (dtype == 0)
        return cw_launch(moe_route_kernel<float>, dim3(N), dim3(128), smem, stream, 1, (const float*)x, Wr, b, tok_seq, sel, wt, W, E, top);
    if (dtype == 1)
        return cw_launch(moe_route_kernel<bf16>, dim3(N), dim3(128), smem, stream, 1, (const bf16*)x, Wr, b, tok_seq, sel, wt, W, E, top);
    return CW_ERR_BAD_DTYPE;
}

// ---- pairs by expert --------------------------------------------------------------------------------
// sel [P] (P = tokens * top; < 0: none) -> offsets [E+1] and order [P]: order[offsets[e] .. offsets[e+1]-1] are
// the pairs of expert e.  The order inside an expert's list is whatever the atomics give; no result depends on
// it (every pair's row is computed by itself and summed per token in choice order).  One block.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ sel, int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ rank,
                 int P, int E) {
    extern __shared__ int count_s[];  // [E + 1]
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) count_s[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = sel[p];
        if (e >= 0 && e < E) rank[p] = atomicAdd(&count_s[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            const int n = count_s[e];
            count_s[e] = run;
            run += n;
        }
        count_s[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = count_s[e];
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = sel[p];
        if (e >= 0 && e < E) order[count_s[e] + rank[p]] = p;
    }
}

extern "C" int cw_moe_group(const int* sel, int* offsets, int* order, int* rank, int P, int E, cudaStream_t stream) {
    if (P < 0 || E <= 0 || E > 8191) return CW_ERR_BAD_SIZE;
    return cw_launch(moe_group_kernel, dim3(1), dim3(1024), (size_t)(E + 1) * sizeof(int), stream, 1, sel, offsets, order, rank, P, E);
}

// resid[n] += sum_t wt[n, t] * y[n * top + t] over the choices in order.
__global__ void __launch_bounds__(256)
moe_combine_kernel(float* __restrict__ resid, const float* __restrict__ y, const int* __restrict__ sel,
                   const float* __restrict__ wt, int W, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    if (sel[(size_t)row * top] < 0) return;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = 0.f;
        for (int t = 0; t < top; ++t) acc = fmaf(wt[(size_t)row * top + t], y[((size_t)row * top + t) * W + c], acc);
        resid[(size_t)row * W + c] += acc;
    }
}

extern "C" int cw_moe_combine(float* resid, const float* y, const int* sel, const float* wt, int N, int W, int top,
                              cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || W <= 0 || top <= 0) return CW_ERR_BAD_SIZE;
    return cw_launch(moe_combine_kernel, dim3(N), dim3(256), 0, stream, 1, resid, y, sel, wt, W, top);
}

CW_TRACE_TU(grouped_gemm)
