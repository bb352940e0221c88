// Two more recurrences over a state of fixed size per request, and the small kernels around them.  Conventions as in
// recurrence.cu: one flat batch of tokens, request s owns rows q_start[s] .. q_start[s+1]-1, its state lives in row
// slots[s] of a float32 table [slots, state_stride], rows whose tok_seq is negative are padding of a fixed-shape step.
//
//   cw_unit_heads          every head of a row divided by sqrt(sum of squares + eps), times a scale (one scale for the
//                          leading heads, another for the rest), in place
//   cw_delta_coefficients  a[t, h, i] = exp(-exp(A[h]) softplus(pre[t, h, i] + dt[h, i])) and beta[t, h] = sigmoid(.), in place
//   cw_delta_scan          the gated delta rule with a decay per key channel:
//                              S <- diag(a_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  y_t = S^T q_t
//   cw_gate_scan           the scalar part of a matrix memory with exponential gates, per request and head in token order:
//                              li = cap tanh((zi + bi)/cap), lf = log sigmoid(cap tanh((zf + bf)/cap)),
//                              m_t = max(lf + m_(t-1), li);  keep = exp(lf + m_(t-1) - m_t), take = exp(li - m_t), floor = exp(-m_t)
//                          written as [keep | take | floor] per token: the coefficients of cw_recurrence_scan's form 4
//   cw_memory_norm         what form 4 leaves per head, [S^T q (dv) | n . q], divided by max(|n . q|, floor) + 1e-6, each
//                          head divided by its root mean square, times a weight, times sigmoid(gate)
//
// Everything here is float32 in both run precisions.
#include "common.cuh"

// ---- unit vectors per head ------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
unit_heads_kernel(float* __restrict__ x, int ld, int N, int heads, int dim, float eps, int heads_a, float scale_a, float scale_b) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // a warp per (row, head)
    if (item >= (long long)N * heads) return;
    const int row = (int)(item / heads), h = (int)(item - (long long)row * heads);
    float* at = x + (size_t)row * ld + (size_t)h * dim;
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) ss = fmaf(at[i], at[i], ss);
    ss = warp_sum(ss);
    const float f = (h < heads_a ? scale_a : scale_b) / sqrtf(ss + eps);
    for (int i = lane; i < dim; i += 32) at[i] *= f;
}

extern "C" int cw_unit_heads(float* x, int ld, int N, int heads, int dim, float eps, int heads_a, float scale_a, float scale_b,
                             cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || heads <= 0 || dim <= 0 || ld < heads * dim) return CW_ERR_BAD_SIZE;
    const long long items = (long long)N * heads;
    return cw_launch_ordered(unit_heads_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, stream, x, ld, N, heads, dim, eps, heads_a,
                             scale_a, scale_b);
}

// ---- decays and write strengths of the delta rule ----------------------------------------------------------
__global__ void __launch_bounds__(256)
delta_coefficients_kernel(float* __restrict__ pre, int ldp, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                          float* __restrict__ beta, int ldb, int N, int H, int Dk) {
    pdl_wait();
    const int C = H * Dk;
    const long long total = (long long)N * (C + H);
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / (C + H)), c = (int)(idx - (long long)t * (C + H));
        if (c < C) {
            float* at = pre + (size_t)t * ldp + c;
            const float x = *at + dt_bias[c];
            const float step = fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
            *at = expf(-expf(a_log[c / Dk]) * step);
        } else {
            float* at = beta + (size_t)t * ldb + (c - C);
            *at = 1.f / (1.f + expf(-*at));
        }
    }
}

extern "C" int cw_delta_coefficients(float* pre, int ldp, const float* dt_bias, const float* a_log, float* beta, int ldb, int N, int H,
                                     int Dk, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || H <= 0 || Dk <= 0 || ldp < H * Dk || ldb < H) return CW_ERR_BAD_SIZE;
    const long long total = (long long)N * (H * Dk + H);
    const int blocks = (int)min((long long)148 * 8, (total + 255) / 256);
    return cw_launch_ordered(delta_coefficients_kernel, dim3(blocks), dim3(256), 0, stream, pre, ldp, dt_bias, a_log, beta, ldb, N, H, Dk);
}

// ---- the delta rule ---------------------------------------------------------------------------------------
// State per request and head: S [Dk, Dv] stored value-column-major (element (i, j) of head h at (h*Dv + j)*Dk + i).
// Blocks: (request, head, slice of JB value columns); IP threads share a value column, a thread owns key channels
// ipart, ipart + IP, ..  The operands of DC tokens at a time are staged in shared memory by cp.async (the next chunk
// while the current one runs).  Per token the column's S^T k is summed over the IP lanes by shuffles (the update needs
// it); the read-out sums wait until the chunk is through.  Every sum has a fixed order, so a row's result does not
// depend on how the request's tokens were cut into steps or on what else the step holds.
#define DS 8    // key channels per thread
#define DC 16   // tokens per staged chunk

__device__ __forceinline__ void dcp4(float* smem, const float* gmem) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gmem) : "memory");
}
__device__ __forceinline__ void dcp16(float* smem, const float* gmem) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem) : "memory");
}

__global__ void __launch_bounds__(256)
delta_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk, const float* __restrict__ v, int ldv,
                  const float* __restrict__ a, int lda, const float* __restrict__ beta, int ldb, float* __restrict__ state,
                  long long state_stride, long long state_off, const long long* __restrict__ slots, const int* __restrict__ tok_seq,
                  const int* __restrict__ q_start, int Dk, int Dv, int heads_per_group, int IP, int wide, float* __restrict__ out,
                  int ldo) {
    extern __shared__ __align__(16) float ds_smem[];
    pdl_wait();
    const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int start = q_start[seq], end = q_start[seq + 1];
    if (end <= start) return;
    const int ipart = tid % IP, jl = tid / IP, JB = blockDim.x / IP;
    const int j0 = blockIdx.z * JB, j = j0 + jl;
    const bool live = j < Dv;
    if (tok_seq[start] < 0) {  // padding rows of a fixed-shape step: no request, no state
        if (live && ipart == 0)
            for (int t = start; t < end; ++t) out[(size_t)t * ldo + (size_t)h * Dv + j] = 0.f;
        return;
    }
    // one buffer: q [DC][Dk], k [DC][Dk], a [DC][Dk], v [DC][JB], beta [DC]
    const int buf_words = 3 * DC * Dk + DC * JB + DC;
    const int g = h / heads_per_group;
    float* S_mem = state + slots[seq] * state_stride + state_off + ((size_t)h * Dv + (live ? j : 0)) * Dk;
    float S[DS];
#pragma unroll
    for (int r = 0; r < DS; ++r) {
        const int i = ipart + r * IP;
        S[r] = (i < Dk && live) ? S_mem[i] : 0.f;
    }
    const float* qp = q + (size_t)g * Dk;
    const float* kp = k + (size_t)g * Dk;
    const float* ap = a + (size_t)h * Dk;
    const float* vp = v + (size_t)h * Dv + j0;
    const float* bp = beta + h;
    const int nv = min(JB, Dv - j0);
    auto fetch = [&](int t0, float* buf) {
        const int n = min(DC, end - t0);
        float* qs = buf;
        float* ks = buf + DC * Dk;
        float* as = buf + 2 * DC * Dk;
        float* vs = buf + 3 * DC * Dk;
        float* bs = vs + DC * JB;
        if (wide) {  // rows of whole 16-byte pieces at 16-byte addresses
            const int pieces = Dk >> 2;
            for (int idx = tid; idx < n * pieces; idx += blockDim.x) {
                const int t = idx / pieces, i = (idx - t * pieces) << 2;
                dcp16(qs + t * Dk + i, qp + (size_t)(t0 + t) * ldq + i);
                dcp16(ks + t * Dk + i, kp + (size_t)(t0 + t) * ldk + i);
                dcp16(as + t * Dk + i, ap + (size_t)(t0 + t) * lda + i);
            }
        } else {
            for (int idx = tid; idx < n * Dk; idx += blockDim.x) {
                const int t = idx / Dk, i = idx - t * Dk;
                dcp4(qs + idx, qp + (size_t)(t0 + t) * ldq + i);
                dcp4(ks + idx, kp + (size_t)(t0 + t) * ldk + i);
                dcp4(as + idx, ap + (size_t)(t0 + t) * lda + i);
            }
        }
        for (int idx = tid; idx < n * nv; idx += blockDim.x) {
            const int t = idx / nv, c = idx - t * nv;
            dcp4(vs + t * JB + c, vp + (size_t)(t0 + t) * ldv + c);
        }
        for (int t = tid; t < n; t += blockDim.x) dcp4(bs + t, bp + (size_t)(t0 + t) * ldb);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(start, ds_smem);
    int which = 0;
    for (int t0 = start; t0 < end; t0 += DC, which ^= 1) {
        const int n = min(DC, end - t0);
        float* buf = ds_smem + which * buf_words;
        const float* qs = buf;
        const float* ks = buf + DC * Dk;
        const float* as = buf + 2 * DC * Dk;
        const float* vs = buf + 3 * DC * Dk;
        const float* bs = vs + DC * JB;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // this chunk has landed; everyone has left the other buffer
        if (t0 + DC < end) fetch(t0 + DC, ds_smem + (which ^ 1) * buf_words);
        float part[DC];
#pragma unroll
        for (int t = 0; t < DC; ++t) {
            part[t] = 0.f;
            if (t < n) {
                float kc[DS], aS[DS];
                float dot0 = 0.f, dot1 = 0.f;  // two chains, added at the end: the same order for every token and batch
#pragma unroll
                for (int r = 0; r < DS; ++r) {
                    const int i = ipart + r * IP;
                    const bool on = i < Dk;
                    kc[r] = on ? ks[t * Dk + i] : 0.f;
                    aS[r] = on ? as[t * Dk + i] * S[r] : 0.f;
                    if (r & 1) dot1 = fmaf(aS[r], kc[r], dot1);
                    else dot0 = fmaf(aS[r], kc[r], dot0);
                }
                float dot = dot0 + dot1;
                for (int o = 1; o < IP; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                const float u = live ? bs[t] * (vs[t * JB + jl] - dot) : 0.f;
                float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                for (int r = 0; r < DS; ++r) {
                    const int i = ipart + r * IP;
                    S[r] = fmaf(kc[r], u, aS[r]);
                    const float qc = i < Dk ? qs[t * Dk + i] : 0.f;
                    if (r & 1) sum1 = fmaf(qc, S[r], sum1);
                    else sum0 = fmaf(qc, S[r], sum0);
                }
                part[t] = sum0 + sum1;
            }
        }
#pragma unroll
        for (int t = 0; t < DC; ++t)
            for (int o = 1; o < IP; o <<= 1) part[t] += __shfl_xor_sync(0xffffffffu, part[t], o);
        if (live && ipart == 0) {
#pragma unroll
            for (int t = 0; t < DC; ++t)
                if (t < n) out[(size_t)(t0 + t) * ldo + (size_t)h * Dv + j] = part[t];
        }
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < DS; ++r) {
            const int i = ipart + r * IP;
            if (i < Dk) S_mem[i] = S[r];
        }
    }
}

// q, k [N, groups*Dk] (head h reads group h / heads_per_group), v [N, H*Dv], a [N, H*Dk] decays, beta [N, H]: float32,
// unit column stride, any row stride.  out [N, H*Dv].
extern "C" int cw_delta_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* a, int lda,
                             const float* beta, int ldb, float* state, long long state_stride, long long state_off,
                             const long long* slots, const int* tok_seq, const int* q_start, int S, int H, int Dk, int Dv,
                             int heads_per_group, float* out, int ldo, cudaStream_t stream) {
    if (S == 0) return CW_OK;
    if (S < 0 || H <= 0 || Dk <= 0 || Dv <= 0 || heads_per_group <= 0 || H % heads_per_group) return CW_ERR_BAD_SIZE;
    if (Dk > 32 * DS || H > 65535) return CW_ERR_UNSUPPORTED;
    int IP = 1;
    while (IP * DS < Dk) IP *= 2;
    int threads = 256;  // more value columns per block share the staged q, k and decays; fewer when a head has few columns
    while (threads > 32 && threads / IP >= 2 * Dv) threads /= 2;
    const int JB = threads / IP;
    dim3 grid(S, H, (Dv + JB - 1) / JB);
    const int wide = Dk % 4 == 0 && ldq % 4 == 0 && ldk % 4 == 0 && lda % 4 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)k & 15) == 0 &&
                     ((uintptr_t)a & 15) == 0;
    const size_t smem = 2 * sizeof(float) * (size_t)(3 * DC * Dk + DC * JB + DC);
    static size_t allowed = 48 << 10;
    if (smem > allowed) {
        const cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    return cw_launch_ordered(delta_scan_kernel, grid, dim3(threads), smem, stream, q, ldq, k, ldk, v, ldv, a, lda, beta, ldb, state,
                             state_stride, state_off, slots, tok_seq, q_start, Dk, Dv, heads_per_group, IP, wide, out, ldo);
}

// ---- the gates of a matrix memory -----------------------------------------------------------------------
// zi, zf [N, ld*] float32 pre-activations of the input and forget gates (a column per head); the running maximum m of
// every head is one float of the request's state (at state_off + h; 0 when a request starts).  coef [N, 3H].
// A block per request, GS_WORDS / H tokens at a time through shared memory, in three passes: every (token, head) pair's
// two logarithms side by side; a thread per head walks the tokens in order (a chain of one addition and one maximum
// per token, its operands already on chip, so a token costs a few cycles); every pair's three exponentials side by
// side.  The chain's order is the tokens' order whatever the cut, so a request's coefficients do not depend on how
// its tokens came in steps.
#define GS_WORDS 2048
__global__ void __launch_bounds__(1024)
gate_scan_kernel(const float* __restrict__ zi, int ldi, const float* __restrict__ zf, int ldf, const float* __restrict__ bias_i,
                 const float* __restrict__ bias_f, float cap, float* __restrict__ state, long long state_stride, long long state_off,
                 const long long* __restrict__ slots, const int* __restrict__ tok_seq, const int* __restrict__ q_start, int H,
                 float* __restrict__ coef) {
    __shared__ float s_li[GS_WORDS], s_lf[GS_WORDS], s_m[2 * GS_WORDS];  // s_m: the maximum before token t at [t][h], after it at [t+1][h]
    pdl_wait();
    const int seq = blockIdx.x;
    const int start = q_start[seq], end = q_start[seq + 1];
    if (end <= start) return;
    const size_t ldc = 3 * (size_t)H;
    if (tok_seq[start] < 0) {  // padding rows: coefficients that leave a zero state at zero
        const int n = end - start;
        for (int idx = threadIdx.x; idx < n * 3 * H; idx += blockDim.x) coef[(size_t)start * ldc + idx] = idx % (3 * H) < 2 * H ? 0.f : 1.f;
        return;
    }
    float* m_mem = state + slots[seq] * state_stride + state_off;
    const int TC = GS_WORDS / H;  // (the launcher refuses more heads than GS_WORDS)
    for (int c0 = start; c0 < end; c0 += TC) {
        const int n = min(TC, end - c0);
        for (int idx = threadIdx.x; idx < n * H; idx += blockDim.x) {
            const int t = c0 + idx / H, h = idx % H;
            const float li = cap * tanhf((zi[(size_t)t * ldi + h] + (bias_i != nullptr ? bias_i[h] : 0.f)) / cap);
            const float c = cap * tanhf((zf[(size_t)t * ldf + h] + (bias_f != nullptr ? bias_f[h] : 0.f)) / cap);
            s_li[idx] = li;
            s_lf[idx] = fminf(c, 0.f) - log1pf(expf(-fabsf(c)));
        }
        __syncthreads();
        for (int h = threadIdx.x; h < H; h += blockDim.x) {
            float m = m_mem[h];
            s_m[h] = m;
            for (int t0 = 0; t0 < n; t0 += 8) {  // eight tokens' operands fetched side by side, then the chain through them
                float li[8], lf[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int at = min(t0 + j, n - 1) * H + h;
                    li[j] = s_li[at];
                    lf[j] = s_lf[at];
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (t0 + j < n) {
                        m = fmaxf(lf[j] + m, li[j]);
                        s_m[(t0 + j + 1) * H + h] = m;
                    }
                }
            }
            m_mem[h] = m;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < n * H; idx += blockDim.x) {
            const int t = idx / H, h = idx - t * H;
            const float before = s_m[idx], after = s_m[idx + H];
            float* c = coef + (size_t)(c0 + t) * ldc;
            c[h] = expf(s_lf[idx] + before - after);
            c[H + h] = expf(s_li[idx] - after);
            c[2 * H + h] = expf(-after);
        }
        __syncthreads();  // the next chunk writes the same shared memory
    }
}

// N: the rows of the step (all requests'), which only sizes the blocks.
extern "C" int cw_gate_scan(const float* zi, int ldi, const float* zf, int ldf, const float* bias_i, const float* bias_f, float cap,
                            float* state, long long state_stride, long long state_off, const long long* slots, const int* tok_seq,
                            const int* q_start, int S, int H, int N, float* coef, cudaStream_t stream) {
    if (S == 0) return CW_OK;
    if (S < 0 || H <= 0 || ldi < H || ldf < H || !(cap > 0.f)) return CW_ERR_BAD_SIZE;
    if (H > GS_WORDS) return CW_ERR_UNSUPPORTED;
    const long long per_request = (long long)(N > 0 ? N : S) * H / S;  // pairs of a request, if the rows were spread evenly
    const int threads = per_request >= 8192 ? 1024 : per_request >= 1024 ? 256 : 128;
    return cw_launch_ordered(gate_scan_kernel, dim3(S), dim3(threads), 0, stream, zi, ldi, zf, ldf, bias_i, bias_f, cap, state, state_stride,
                             state_off, slots, tok_seq, q_start, H, coef);
}

// ---- read-out of the matrix memory ------------------------------------------------------------------------
// y [N, H*(dv+1)] float32: per head [S^T q (dv) | n . q];  floor_ [N, ldfl] (a column per head);  gate z [N, ldz];
// weight [H*dv].  out[row, h*dv + c] = rmsnorm_head(y_c / (max(|n . q|, floor) + 1e-6)) * weight * sigmoid(z).
// A warp per (row, head).
template <typename T>
__global__ void __launch_bounds__(256)
memory_norm_kernel(const float* __restrict__ y, const float* __restrict__ floor_, int ldfl, const float* __restrict__ z, int ldz,
                   const float* __restrict__ weight, T* __restrict__ out, int N, int H, int dv, float eps) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)N * H) return;
    const int row = (int)(item / H), h = (int)(item - (long long)row * H);
    const float* yr = y + ((size_t)row * H + h) * (dv + 1);
    const float inv_d = 1.f / (fmaxf(fabsf(yr[dv]), floor_[(size_t)row * ldfl + h]) + 1e-6f);
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) {
        const float u = yr[c] * inv_d;
        ss = fmaf(u, u, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    const float* zr = z + (size_t)row * ldz + (size_t)h * dv;
    const float* wr = weight + (size_t)h * dv;
    T* o = out + ((size_t)row * H + h) * dv;
    for (int c = lane; c < dv; c += 32) o[c] = from_f<T>(yr[c] * inv_d * inv * wr[c] / (1.f + expf(-zr[c])));
}

extern "C" int cw_memory_norm(const float* y, const float* floor_, int ldfl, const float* z, int ldz, const float* weight, void* out,
                              int N, int H, int dv, float eps, int dtype, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || H <= 0 || dv <= 0 || ldfl < H || ldz < H * dv) return CW_ERR_BAD_SIZE;
    const long long items = (long long)N * H;
    const dim3 grid((unsigned)((items + 7) / 8));
    if (dtype == 0)
        return cw_launch_ordered(memory_norm_kernel<float>, grid, dim3(256), 0, stream, y, floor_, ldfl, z, ldz, weight, (float*)out, N, H,
                                 dv, eps);
    if (dtype == 1)
        return cw_launch_ordered(memory_norm_kernel<bf16>, grid, dim3(256), 0, stream, y, floor_, ldfl, z, ldz, weight, (bf16*)out, N, H, dv,
                                 eps);
    return CW_ERR_BAD_DTYPE;
}

CW_TRACE_TU(recurrence_gated)
