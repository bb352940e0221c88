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
// Beside it the router of a mixture of experts (float32 logits, the `top` largest, weighted by the softmax
// over the chosen or by their shares of the softmax over all; optionally only experts of the best runs of
// neighbours), the grouping of (token, choice) pairs by expert, and the weighted sum of the experts'
// outputs into the float32 residual, in choice order.
#include "common.cuh"

#define GG_TM 32
#define GG_TN 64
#define GG_TK 32

#define GG_EPI_STORE 0        // C (T) = acc
#define GG_EPI_STORE_F32 1    // C (float) = acc
#define GG_EPI_SILU_MUL 2     // C (T) = silu(acc) * acc2, acc2 from B2; with a positive `glu_limit` the clamped form below
#define GG_EPI_SIGMOID_GATE 3 // C (T) = acc * sigmoid(gate[dst, c_group_off*g + n])

// The gated activation of the two-product form: silu(a) b, or, with a positive limit,
//   a' = min(a, limit), b' = clamp(b, -limit, limit):  a' sigmoid(1.702 a') (b' + 1)
__device__ __forceinline__ float gg_glu(float a, float b, float limit) {
    if (limit > 0.f) {
        a = fminf(a, limit);
        b = fminf(fmaxf(b, -limit), limit);
        return a / (1.f + expf(-1.702f * a)) * (b + 1.f);
    }
    return a / (1.f + expf(-a)) * b;
}

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const T* __restrict__ A, int lda, int a_group_off, const T* __restrict__ B, const T* __restrict__ B2,
                    long long b_stride, void* __restrict__ Cv, int ldc, int c_group_off,
                    const int* __restrict__ offsets, const int* __restrict__ a_index, int a_div,
                    const int* __restrict__ c_index, const T* __restrict__ gate, int ldg,
                    int M, int Nout, int K, int G, float glu_limit) {
    __shared__ float As[GG_TK][GG_TM + 1];
    __shared__ float Bs[GG_TK][GG_TN + 1];
    __shared__ float B2s[EPI == GG_EPI_SILU_MUL ? GG_TK : 1][GG_TN + 1];
    __shared__ int src_s[GG_TM], dst_s[GG_TM];
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
                if (EPI == GG_EPI_SILU_MUL) v = gg_glu(v, acc2[r][c], glu_limit);
                if (EPI == GG_EPI_SIGMOID_GATE) v = v / (1.f + expf(-to_f(gate[(size_t)d * ldg + (size_t)g * c_group_off + n])));
                ((T*)Cv)[at] = from_f<T>(v);
            }
        }
    }
}

// ---- the same product on the tensor cores (bfloat16 operands, float32 accumulation) -------------------
// Tiles of 64 rows x 128 outputs, K in steps of 32 through a three-stage cp.async ring, eight warps of
// 32 x 32 outputs each on mma.sync m16n8k16.  A's rows are gathered through the index as they are
// fetched.  Needs K, the row strides and the per-group offsets to be multiples of 8 elements (16-byte
// copies); otherwise the kernel above runs.  A tile of few rows (single tokens) costs what its weights
// cost to stream.
#define GM_TM 64
#define GM_TN 128
#define GM_TK 32
#define GM_LD 40  // padded row of a stage, in elements: 80 bytes, so that eight rows fall into distinct banks
#define GM_STAGES 3

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int EPI>
__global__ void __launch_bounds__(256)
grouped_gemm_mma_kernel(const bf16* __restrict__ A, int lda, int a_group_off, const bf16* __restrict__ B,
                        const bf16* __restrict__ B2, long long b_stride, void* __restrict__ Cv, int ldc, int c_group_off,
                        const int* __restrict__ offsets, const int* __restrict__ a_index, int a_div,
                        const int* __restrict__ c_index, const bf16* __restrict__ gate, int ldg,
                        int M, int Nout, int K, int G, float glu_limit) {
    extern __shared__ __align__(16) unsigned char gm_smem[];
    constexpr bool TWO = EPI == GG_EPI_SILU_MUL;
    bf16* As = (bf16*)gm_smem;                       // [stages][TM][LD]
    bf16* Bs = As + GM_STAGES * GM_TM * GM_LD;       // [stages][TN][LD]
    bf16* B2s = Bs + GM_STAGES * GM_TN * GM_LD;      // [stages][TN][LD] (two-product form only)
    __shared__ int src_s[GM_TM], dst_s[GM_TM];
    pdl_wait();
    int g, row0, rows_end;
    if (offsets == nullptr) {
        const int tiles = (M + GM_TM - 1) / GM_TM;
        g = blockIdx.x / tiles;
        row0 = (blockIdx.x % tiles) * GM_TM;
        rows_end = M;
    } else {
        int tile = blockIdx.x;
        g = 0;
        while (g < G) {
            const int n = offsets[g + 1] - offsets[g];
            const int t = (n + GM_TM - 1) / GM_TM;
            if (tile < t) break;
            tile -= t;
            ++g;
        }
        if (g >= G) return;
        row0 = offsets[g] + tile * GM_TM;
        rows_end = offsets[g + 1];
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < GM_TM) {
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
    const int n0 = blockIdx.y * GM_TN;
    const bf16* Bg = B + (size_t)g * b_stride;
    const bf16* B2g = TWO ? B2 + (size_t)g * b_stride : nullptr;
    const int KT = (K + GM_TK - 1) / GM_TK;
    auto load = [&](int kt, int stage) {
        {
            const int row = tid >> 2, k = kt * GM_TK + (tid & 3) * 8;
            const int s = src_s[row];
            const bool on = s >= 0 && k < K;
            cp_async16(As + ((size_t)stage * GM_TM + row) * GM_LD + (tid & 3) * 8,
                       on ? A + (size_t)s * lda + (size_t)g * a_group_off + k : A, on);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + i * 256;
            const int n = idx >> 2, k = kt * GM_TK + (idx & 3) * 8;
            const bool on = n0 + n < Nout && k < K;
            const size_t at = ((size_t)stage * GM_TN + n) * GM_LD + (idx & 3) * 8;
            cp_async16(Bs + at, on ? Bg + (size_t)(n0 + n) * K + k : Bg, on);
            if (TWO) cp_async16(B2s + at, on ? B2g + (size_t)(n0 + n) * K + k : B2g, on);
        }
    };
    const int wm = warp >> 2, wn = warp & 3;  // 2 x 4 warps, 32 x 32 outputs each
    float acc[2][4][4] = {}, acc2[TWO ? 2 : 1][TWO ? 4 : 1][4] = {};
#pragma unroll
    for (int s = 0; s < GM_STAGES - 1; ++s) {
        if (s < KT) load(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < KT; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(GM_STAGES - 2) : "memory");
        __syncthreads();  // stage kt has landed for everyone, and everyone is done with stage kt-1
        if (kt + GM_STAGES - 1 < KT) load(kt + GM_STAGES - 1, (kt + GM_STAGES - 1) % GM_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int stage = kt % GM_STAGES;
        const bf16* as = As + (size_t)stage * GM_TM * GM_LD;
        const bf16* bs = Bs + (size_t)stage * GM_TN * GM_LD;
        const bf16* b2s = B2s + (size_t)stage * GM_TN * GM_LD;
#pragma unroll
        for (int kk = 0; kk < GM_TK; kk += 16) {
            unsigned a[2][4];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
                ldmatrix_x4(a[mi], as + (size_t)(wm * 32 + mi * 16 + (lane & 15)) * GM_LD + kk + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < 2; ++np) {  // two n-tiles of 8 per ldmatrix
                const size_t at = (size_t)(wn * 32 + np * 16 + (lane & 7) + (lane >> 4) * 8) * GM_LD + kk + ((lane >> 3) & 1) * 8;
                unsigned b[4];
                ldmatrix_x4(b, bs + at);
#pragma unroll
                for (int mi = 0; mi < 2; ++mi) {
                    mma_bf16(acc[mi][np * 2], a[mi], b[0], b[1]);
                    mma_bf16(acc[mi][np * 2 + 1], a[mi], b[2], b[3]);
                }
                if (TWO) {
                    ldmatrix_x4(b, b2s + at);
#pragma unroll
                    for (int mi = 0; mi < 2; ++mi) {
                        mma_bf16(acc2[TWO ? mi : 0][TWO ? np * 2 : 0], a[mi], b[0], b[1]);
                        mma_bf16(acc2[TWO ? mi : 0][TWO ? np * 2 + 1 : 0], a[mi], b[2], b[3]);
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int d = dst_s[wm * 32 + mi * 16 + half * 8 + (lane >> 2)];
            if (d < 0) continue;
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int n = n0 + wn * 32 + ni * 8 + (lane & 3) * 2 + e;
                    if (n >= Nout) continue;
                    const size_t at = (size_t)d * ldc + (size_t)g * c_group_off + n;
                    float v = acc[mi][ni][half * 2 + e];
                    if (EPI == GG_EPI_STORE_F32) {
                        ((float*)Cv)[at] = v;
                    } else {
                        if (TWO) v = gg_glu(v, acc2[TWO ? mi : 0][TWO ? ni : 0][half * 2 + e], glu_limit);
                        if (EPI == GG_EPI_SIGMOID_GATE)
                            v = v / (1.f + expf(-to_f(gate[(size_t)d * ldg + (size_t)g * c_group_off + n])));
                        ((bf16*)Cv)[at] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
    }
}

template <int EPI>
static int launch_grouped_mma(dim3 grid, cudaStream_t stream, const void* A, int lda, int a_group_off, const void* B, const void* B2,
                              long long b_stride, void* C, int ldc, int c_group_off, const int* offsets, const int* a_index,
                              int a_div, const int* c_index, const void* gate, int ldg, int M, int Nout, int K, int G, float glu_limit) {
    const size_t smem = (size_t)GM_STAGES * (GM_TM + (EPI == GG_EPI_SILU_MUL ? 2 : 1) * GM_TN) * GM_LD * sizeof(bf16);
    static bool configured = false;  // (per instantiation)
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(grouped_gemm_mma_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return cw_launch_ordered(grouped_gemm_mma_kernel<EPI>, grid, dim3(256), smem, stream, (const bf16*)A, lda, a_group_off, (const bf16*)B,
                     (const bf16*)B2, b_stride, C, ldc, c_group_off, offsets, a_index, a_div, c_index, (const bf16*)gate, ldg, M, Nout,
                     K, G, glu_limit);
}

static int g_grouped_mma = 1;
extern "C" int cw_grouped_gemm_set_mma(int on) { g_grouped_mma = on ? 1 : 0; return CW_OK; }

template <typename T>
static int launch_grouped(int epi, dim3 grid, cudaStream_t stream, const void* A, int lda, int a_group_off, const void* B,
                          const void* B2, long long b_stride, void* C, int ldc, int c_group_off, const int* offsets,
                          const int* a_index, int a_div, const int* c_index, const void* gate, int ldg, int M, int Nout, int K,
                          int G, float glu_limit) {
#define GG_GO(E)                                                                                                              \
    return cw_launch_ordered(grouped_gemm_kernel<T, E>, grid, dim3(256), 0, stream, (const T*)A, lda, a_group_off, (const T*)B,    \
                     (const T*)B2, b_stride, C, ldc, c_group_off, offsets, a_index, a_div, c_index, (const T*)gate, ldg, M,   \
                     Nout, K, G, glu_limit)
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
                               float glu_limit, int dtype, cudaStream_t stream) {
    if (M == 0) return CW_OK;
    if (M < 0 || Nout <= 0 || K <= 0 || G <= 0 || a_div <= 0) return CW_ERR_BAD_SIZE;
    if (epilogue == GG_EPI_SILU_MUL && B2 == nullptr) return CW_ERR_BAD_SIZE;
    if (epilogue == GG_EPI_SIGMOID_GATE && gate == nullptr) return CW_ERR_BAD_SIZE;
    const long long tiles = offsets == nullptr ? (long long)G * ((M + GG_TM - 1) / GG_TM) : (long long)(M + GG_TM - 1) / GG_TM + G;
    if (tiles > 0x7fffffffLL) return CW_ERR_UNSUPPORTED;
    dim3 grid((unsigned)tiles, (Nout + GG_TN - 1) / GG_TN);
    if (dtype == 0)
        return launch_grouped<float>(epilogue, grid, stream, A, lda, a_group_off, B, B2, b_stride, C, ldc, c_group_off, offsets,
                                     a_index, a_div, c_index, gate, ldg, M, Nout, K, G, glu_limit);
    const bool aligned = K % 8 == 0 && lda % 8 == 0 && a_group_off % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)B & 15) == 0 &&
                         ((uintptr_t)B2 & 15) == 0;
    if (dtype == 1 && g_grouped_mma && aligned) {
        const long long mtiles = offsets == nullptr ? (long long)G * ((M + GM_TM - 1) / GM_TM) : (long long)(M + GM_TM - 1) / GM_TM + G;
        dim3 mgrid((unsigned)mtiles, (Nout + GM_TN - 1) / GM_TN);
#define GM_GO(E)                                                                                                                 \
    return launch_grouped_mma<E>(mgrid, stream, A, lda, a_group_off, B, B2, b_stride, C, ldc, c_group_off, offsets, a_index, a_div, \
                                 c_index, gate, ldg, M, Nout, K, G, glu_limit)
        switch (epilogue) {
            case GG_EPI_STORE: GM_GO(GG_EPI_STORE);
            case GG_EPI_STORE_F32: GM_GO(GG_EPI_STORE_F32);
            case GG_EPI_SILU_MUL: GM_GO(GG_EPI_SILU_MUL);
            case GG_EPI_SIGMOID_GATE: GM_GO(GG_EPI_SIGMOID_GATE);
        }
#undef GM_GO
        return CW_ERR_UNSUPPORTED;
    }
    if (dtype == 1)
        return launch_grouped<bf16>(epilogue, grid, stream, A, lda, a_group_off, B, B2, b_stride, C, ldc, c_group_off, offsets,
                                    a_index, a_div, c_index, gate, ldg, M, Nout, K, G, glu_limit);
    return CW_ERR_BAD_DTYPE;
}

// ---- router ---------------------------------------------------------------------------------------
// logits [N, E] float32 (a product with float32 accumulation, made by the caller) + bias; the `top`
// largest (the lower index wins a tie).  sel < 0 marks a padding row.  A warp per token.
//   mode 0: weights = softmax over the chosen logits.
//   mode 1: scores = softmax over all E logits; weights = the chosen experts' scores as they are.
//   mode 2: scores = sigmoid of each logit; experts are ranked by score + correction[e] (`correction` null: by the score),
//           weights = the chosen experts' scores without the correction.
// Every weight is multiplied by weight_scale at the end.
// groups > 1: the experts lie in `groups` equal runs of neighbours; a run counts as the sum of its `group_rank` largest
// entries (1: its largest entry), and only experts of the `keep` best runs can be chosen (the others count as minus
// infinity, whatever the sign of the entries).
__global__ void __launch_bounds__(128)
moe_choose_kernel(const float* __restrict__ logits, const float* __restrict__ b, const int* __restrict__ tok_seq,
                  int* __restrict__ sel, float* __restrict__ wt, int N, int E, int top, int mode, int groups, int keep,
                  const float* __restrict__ correction, float weight_scale, int group_rank) {
    extern __shared__ float choose_s[];  // per warp: [E] logits or scores, [top] chosen ones, [groups] the runs' best, [E] plain scores
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * 4 + warp;
    if (row >= N) return;
    if (tok_seq[row] < 0) {
        for (int t = lane; t < top; t += 32) {
            sel[(size_t)row * top + t] = -1;
            wt[(size_t)row * top + t] = 0.f;
        }
        return;
    }
    float* logit_s = choose_s + (size_t)warp * (2 * E + top + groups);
    float* chosen_s = logit_s + E;
    float* group_s = chosen_s + top;
    float* score_s = group_s + groups;  // mode 2: the scores that become weights
    for (int e = lane; e < E; e += 32) logit_s[e] = logits[(size_t)row * E + e] + (b != nullptr ? b[e] : 0.f);
    __syncwarp();
    if (mode == 1) {  // every expert's share of the softmax over all of them (sums in a fixed order)
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, logit_s[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) sum += expf(logit_s[e] - mx);
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) logit_s[e] = expf(logit_s[e] - mx) / sum;
        __syncwarp();
    }
    if (mode == 2) {
        for (int e = lane; e < E; e += 32) {
            const float sc = 1.f / (1.f + expf(-logit_s[e]));
            score_s[e] = sc;
            logit_s[e] = sc + (correction != nullptr ? correction[e] : 0.f);
        }
        __syncwarp();
    }
    if (groups > 1) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float rank = 0.f;
            int taken[4] = {-1, -1, -1, -1};  // (group_rank <= 4)
            for (int r = 0; r < group_rank; ++r) {  // the largest entries one by one, the lower index first among equals
                float best = -INFINITY;
                int at = -1;
                for (int e = g * per; e < (g + 1) * per; ++e) {
                    bool used = false;
                    for (int u = 0; u < r; ++u) used = used || taken[u] == e;
                    if (!used && (at < 0 || logit_s[e] > best)) best = logit_s[e], at = e;
                }
                taken[r] = at;
                rank = r == 0 ? best : rank + best;
            }
            group_s[g] = rank;
        }
        __syncwarp();
        for (int t = 0; t < keep; ++t) {  // the best runs one by one; a kept run is marked with +inf
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float v = group_s[g];
                if (v != INFINITY && v > best) best = v, at = g;
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ov > best || (ov == best && oa < at)) best = ov, at = oa;
            }
            if (lane == 0 && at != 0x7fffffff) group_s[at] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (group_s[e / per] != INFINITY) logit_s[e] = -INFINITY;
        __syncwarp();
    }
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
        if (at == 0x7fffffff) at = t % E;  // no finite entry left (never with finite inputs and enough allowed experts)
        if (lane == 0) {
            sel[(size_t)row * top + t] = at;
            chosen_s[t] = best;
            logit_s[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (mode == 1) {
        for (int t = lane; t < top; t += 32) wt[(size_t)row * top + t] = chosen_s[t] == -INFINITY ? 0.f : chosen_s[t] * weight_scale;
        return;
    }
    if (mode == 2) {
        for (int t = lane; t < top; t += 32) {
            const int e = sel[(size_t)row * top + t];  // (written by lane 0 above, made visible by __syncwarp)
            wt[(size_t)row * top + t] = chosen_s[t] == -INFINITY ? 0.f : score_s[e] * weight_scale;
        }
        return;
    }
    const float first = chosen_s[0];
    float total = 0.f;
    for (int t = 0; t < top; ++t) total += expf(chosen_s[t] - first);  // the same order in every lane
    for (int t = lane; t < top; t += 32) wt[(size_t)row * top + t] = expf(chosen_s[t] - first) / total * weight_scale;
}

extern "C" int cw_moe_choose(const float* logits, const float* b, const int* tok_seq, int* sel, float* wt, int N, int E, int top,
                             int mode, int groups, int keep, const float* correction, float weight_scale, int group_rank,
                             cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || E <= 0 || top <= 0 || top > E || mode < 0 || mode > 2) return CW_ERR_BAD_SIZE;
    if (groups < 1 || E % groups || keep < 1 || keep > groups || (long long)keep * (E / groups) < top) return CW_ERR_BAD_SIZE;
    if (group_rank < 1 || group_rank > 4 || group_rank > E / groups) return CW_ERR_BAD_SIZE;
    const size_t smem = 4 * (size_t)(2 * E + top + groups) * sizeof(float);
    if (smem > (48 << 10)) return CW_ERR_UNSUPPORTED;
    return cw_launch_ordered(moe_choose_kernel, dim3((N + 3) / 4), dim3(128), smem, stream, logits, b, tok_seq, sel, wt, N, E, top,
                             mode, groups, keep, correction, weight_scale, group_rank);
}

// ---- pairs by expert --------------------------------------------------------------------------------
// sel [P] (P = tokens * top; < 0: none) -> offsets [E+1] and order [P]: order[offsets[e] .. offsets[e+1]-1] are
// the pairs of expert e.  The order inside an expert's list is whatever the atomics give; no result depends on
// it (every pair's row is computed by itself and summed per token in choice order).  One block.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ sel, int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ rank,
                 int P, int E) {
    extern __shared__ int count_s[];  // [E + 1]
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
    return cw_launch_ordered(moe_group_kernel, dim3(1), dim3(1024), (size_t)(E + 1) * sizeof(int), stream, sel, offsets, order, rank, P, E);
}

// resid[n] += sum_t wt[n, t] * y[n * top + t] over the choices in order; with `assign` the sum replaces resid[n] (rows of no
// request: zeros).
__global__ void __launch_bounds__(256)
moe_combine_kernel(float* __restrict__ resid, const float* __restrict__ y, const int* __restrict__ sel,
                   const float* __restrict__ wt, int W, int top, int assign) {
    pdl_wait();
    const int row = blockIdx.x;
    if (sel[(size_t)row * top] < 0) {
        if (assign)
            for (int c = threadIdx.x; c < W; c += blockDim.x) resid[(size_t)row * W + c] = 0.f;
        return;
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = 0.f;
        for (int t = 0; t < top; ++t) acc = fmaf(wt[(size_t)row * top + t], y[((size_t)row * top + t) * W + c], acc);
        resid[(size_t)row * W + c] = assign ? acc : resid[(size_t)row * W + c] + acc;
    }
}

extern "C" int cw_moe_combine(float* resid, const float* y, const int* sel, const float* wt, int N, int W, int top, int assign,
                              cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || W <= 0 || top <= 0) return CW_ERR_BAD_SIZE;
    return cw_launch_ordered(moe_combine_kernel, dim3(N), dim3(256), 0, stream, resid, y, sel, wt, W, top, assign);
}

CW_TRACE_TU(grouped_gemm)
