// Layers that carry a state of fixed size from token to token instead of a cache of keys: the
// pieces that a state-space layer (Mamba-2 form) and a linear-attention layer with per-channel decay
// (RWKV form) are put together from.  Every kernel takes one flat batch of tokens (prompt portions
// beside single decoded tokens): request s owns rows q_start[s] .. q_start[s+1]-1, its state lives in
// row slots[s] of a float32 table [slots, state_stride], and a portion continues from whatever the
// step before left there.  Rows whose tok_seq is negative are padding of a fixed-shape step.
//
//   cw_shift_mix        m_s = x + (x_prev - x) * mu_s for several mu at once; x_prev of a portion's
//                       first row is the row that cw_carry_rows kept
//   cw_causal_conv      per-channel causal convolution over the last `taps` inputs, bias, SiLU; the
//                       inputs before a portion's first row are the rows that cw_carry_rows kept
//   cw_carry_rows       keeps the last R rows of each request's portion for the next step
//   cw_recurrence_scan  S <- diag(a_t) S + k_t v_t^T, y_t = S^T q_t, in the two forms named below,
//                       float32 state, one pass over the portion in token order
//   cw_gated_group_norm y (*silu(z)) divided by its root mean square in equal parts, times a weight
//                       (times silu(z)): the gate before or after the norm
//   cw_activation       gelu (tanh form), tanh, silu, sigmoid, in place (cw_activation_cols: on some columns of wider rows)
//
// Everything that enters the recurrence (decays, step sizes, the state, the norm) is float32 in both
// run precisions; T only names the type of activations that matrix products read or wrote.
#include "common.cuh"

// ---- token shift ----------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
shift_mix_kernel(const T* __restrict__ x, const float* __restrict__ mu, const float* __restrict__ state,
                 long long state_stride, long long state_off, const long long* __restrict__ slots,
                 const int* __restrict__ tok_seq, const int* __restrict__ q_start, T* __restrict__ out,
                 int N, int W, int mixes) {
    pdl_wait();
    const int row = blockIdx.x;
    const int seq = tok_seq[row];
    const size_t plane = (size_t)N * W;
    if (seq < 0) {
        for (int c = threadIdx.x; c < W; c += blockDim.x)
            for (int s = 0; s < mixes; ++s) out[s * plane + (size_t)row * W + c] = from_f<T>(0.f);
        return;
    }
    const bool first = row == q_start[seq];
    const float* kept = state + slots[seq] * state_stride + state_off;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float cur = to_f(x[(size_t)row * W + c]);
        const float prev = first ? kept[c] : to_f(x[(size_t)(row - 1) * W + c]);
        const float d = prev - cur;
        for (int s = 0; s < mixes; ++s)
            out[s * plane + (size_t)row * W + c] = from_f<T>(fmaf(d, mu[(size_t)s * W + c], cur));
    }
}

extern "C" int cw_shift_mix(const void* x, const float* mu, const float* state, long long state_stride,
                            long long state_off, const long long* slots, const int* tok_seq, const int* q_start,
                            void* out, int N, int W, int mixes, int dtype, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || W <= 0 || mixes <= 0) return CW_ERR_BAD_SIZE;
    if (dtype == 0)
        return cw_launch_ordered(shift_mix_kernel<float>, dim3(N), dim3(256), 0, stream, (const float*)x, mu, state, state_stride,
                         state_off, slots, tok_seq, q_start, (float*)out, N, W, mixes);
    if (dtype == 1)
        return cw_launch_ordered(shift_mix_kernel<bf16>, dim3(N), dim3(256), 0, stream, (const bf16*)x, mu, state, state_stride,
                         state_off, slots, tok_seq, q_start, (bf16*)out, N, W, mixes);
    return CW_ERR_BAD_DTYPE;
}

// ---- short causal convolution ---------------------------------------------------------------------
// x [N, ldx] float32 (a column slice of a wider matrix), weight [C, taps] with the current token's tap
// last, out [N, C] float32 = silu(bias + sum_j weight[c][j] * x[row - (taps-1-j)][c]).
__global__ void __launch_bounds__(256)
causal_conv_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ weight, const float* __restrict__ bias,
                   const float* __restrict__ state, long long state_stride, long long state_off,
                   const long long* __restrict__ slots, const int* __restrict__ tok_seq, const int* __restrict__ q_start,
                   float* __restrict__ out, int C, int taps) {
    pdl_wait();
    const int row = blockIdx.x;
    const int seq = tok_seq[row];
    if (seq < 0) {
        for (int c = threadIdx.x; c < C; c += blockDim.x) out[(size_t)row * C + c] = 0.f;
        return;
    }
    const int start = q_start[seq];
    const int R = taps - 1;
    const float* kept = state + slots[seq] * state_stride + state_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = bias != nullptr ? bias[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int src = row - (R - j);
            const float v = src >= start ? x[(size_t)src * ldx + c] : kept[(size_t)(R - (start - src)) * C + c];
            acc = fmaf(weight[(size_t)c * taps + j], v, acc);
        }
        out[(size_t)row * C + c] = acc / (1.f + expf(-acc));
    }
}

extern "C" int cw_causal_conv(const float* x, int ldx, const float* weight, const float* bias, const float* state,
                              long long state_stride, long long state_off, const long long* slots, const int* tok_seq,
                              const int* q_start, float* out, int N, int C, int taps, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || C <= 0 || taps <= 0 || ldx < C) return CW_ERR_BAD_SIZE;
    return cw_launch_ordered(causal_conv_kernel, dim3(N), dim3(256), 0, stream, x, ldx, weight, bias, state, state_stride, state_off,
                     slots, tok_seq, q_start, out, C, taps);
}

// ---- the rows a later step reads again --------------------------------------------------------------
// kept[R][C] of a request: kept[R-d] is the row d places before the request's next token.  A portion of
// n rows shifts the older rows up by n and appends its own last min(n, R).
template <typename T>
__global__ void __launch_bounds__(256)
carry_rows_kernel(const T* __restrict__ x, int ldx, float* __restrict__ state, long long state_stride,
                  long long state_off, const long long* __restrict__ slots, const int* __restrict__ tok_seq,
                  const int* __restrict__ q_start, int C, int R) {
    pdl_wait();
    const int seq = blockIdx.x;
    const int start = q_start[seq], end = q_start[seq + 1];
    const int n = end - start;
    if (n <= 0 || tok_seq[start] < 0) return;
    float* kept = state + slots[seq] * state_stride + state_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        for (int d = R; d >= 1; --d)  // ascending writes; what is read lies ahead of what was written
            kept[(size_t)(R - d) * C + c] = d <= n ? to_f(x[(size_t)(end - d) * ldx + c]) : kept[(size_t)(R - (d - n)) * C + c];
    }
}

extern "C" int cw_carry_rows(const void* x, int ldx, float* state, long long state_stride, long long state_off,
                             const long long* slots, const int* tok_seq, const int* q_start, int S, int C, int R, int dtype,
                             cudaStream_t stream) {
    if (S == 0 || R == 0) return CW_OK;
    if (S < 0 || C <= 0 || R < 0 || ldx < C) return CW_ERR_BAD_SIZE;
    dim3 grid(S, min(64, (C + 255) / 256));
    if (dtype == 0)
        return cw_launch_ordered(carry_rows_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, ldx, state, state_stride,
                         state_off, slots, tok_seq, q_start, C, R);
    if (dtype == 1)
        return cw_launch_ordered(carry_rows_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)x, ldx, state, state_stride,
                         state_off, slots, tok_seq, q_start, C, R);
    return CW_ERR_BAD_DTYPE;
}

// ---- the recurrence ---------------------------------------------------------------------------------
// Per request and head a state S [Dk, Dv] (float32, stored value-column-major: element (i, j) of head h at
// (h*Dv + j)*Dk + i).  Two forms:
//   FORM 0 (decay per key channel, output before the update, bonus for the current token):
//       y_j = sum_i q_i (S_ij + p1_i k_i v_j);  S_ij <- a_i S_ij + k_i v_j          (coef = a [N, H*Dk])
//   FORM 1 (one decay per head from a step size, output after the update, skip term):
//       S_ij <- a S_ij + dt k_i v_j;  y_j = sum_i q_i S_ij + p2 v_j                  (coef = [a | dt] [N, 2H])
//   FORM 2 (decay per key channel, output after the update):
//       S_ij <- a_i S_ij + k_i v_j;  y_j = q_scale sum_i q_i S_ij                   (coef = a [N, H*Dk])
//   FORM 3 (one constant decay per head, output after the update):
//       S_ij <- p0_h S_ij + k_i v_j;  y_j = q_scale sum_i q_i S_ij                  (no coefficients)
//   FORM 4 (form 1 without the skip term, its coefficients made elsewhere, and one more value column than v has,
//           whose input is 1 for every token: that column of S is the decayed sum of the scaled keys):
//       S_ij <- a S_ij + b k_i v_j;  y_j = q_scale sum_i q_i S_ij,  v_(Dv-1) = 1     (coef = [a | b] [N, >= 2H]; v [N, H*(Dv-1)])
// with the coefficients from cw_recurrence_coefficients (forms 0 and 1), cw_sigmoid_power_decay (form 2) or
// cw_gate_scan (form 4).
// q and k of head h are those of group h / heads_per_group.  Blocks: (request, head, slice of value columns).
// What the recurrence multiplies by, computed once per token before the scan (float32):
//   FORM 0: a[t, c] = exp(-exp(pre[t, c] + p0[c])) for the H*Dk channels, in place
//   FORM 1: dt = softplus(pre[t, h] + p0[h]) (no threshold), out[t, h] = exp(-exp(p1[h]) dt), out[t, H + h] = dt
__global__ void __launch_bounds__(256)
recurrence_coefficients_kernel(int form, float* __restrict__ pre, int ldp, const float* __restrict__ p0,
                               const float* __restrict__ p1, float* __restrict__ out, int N, int C) {
    pdl_wait();
    const long long total = (long long)N * C;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / C), c = (int)(idx - (long long)t * C);
        if (form == 0) {
            float* at = pre + (size_t)t * ldp + c;
            *at = expf(-expf(*at + p0[c]));
        } else {
            const float x = pre[(size_t)t * ldp + c] + p0[c];
            const float dt = fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
            out[(size_t)t * 2 * C + c] = expf(-expf(p1[c]) * dt);
            out[(size_t)t * 2 * C + C + c] = dt;
        }
    }
}

extern "C" int cw_recurrence_coefficients(int form, float* pre, int ldp, const float* p0, const float* p1, float* out, int N, int C,
                                          cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || C <= 0 || ldp < C || (form != 0 && form != 1)) return CW_ERR_BAD_SIZE;
    const long long total = (long long)N * C;
    const int blocks = (int)min((long long)148 * 8, (total + 255) / 256);
    return cw_launch_ordered(recurrence_coefficients_kernel, dim3(blocks), dim3(256), 0, stream, form, pre, ldp, p0, p1, out, N, C);
}

#define RS 8    // key channels per thread
#define RC 16   // tokens per staged chunk

__device__ __forceinline__ void cp_async16f(float* smem, const float* gmem) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async4(float* smem, const float* gmem) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gmem) : "memory");
}

// The operands of RC tokens at a time are copied into shared memory (cp.async, the next chunk while the
// current one is computed) and read from there by the IP x JB threads; a thread owns key channels ipart, ipart + IP, ..
// of value column j, so that neighbouring lanes read neighbouring words of shared memory and of the state.
// The per-token sums over key channels are reduced over the IP lanes of a column after the chunk's loop.
template <int FORM, bool VEC>
__global__ void __launch_bounds__(256)
recurrence_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                       const float* __restrict__ v, int ldv, const float* __restrict__ pre, int ldp,
                       const float* __restrict__ p0, const float* __restrict__ p1, const float* __restrict__ p2,
                       float* __restrict__ state, long long state_stride, long long state_off,
                       const long long* __restrict__ slots, const int* __restrict__ tok_seq,
                       const int* __restrict__ q_start, int Dk, int Dv, int heads_per_group, int IP, int wide, int H,
                       float* __restrict__ out, int ldo, float q_scale) {
    extern __shared__ __align__(16) float rs_smem[];
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
    // one buffer: q [RC][Dk], k [RC][Dk], a [RC][Dk] (forms 0 and 2) or a, dt [2][RC] (FORM 1) or nothing (FORM 3), v [RC][JB]
    constexpr bool CH = FORM == 0 || FORM == 2;  // a decay per key channel and token
    constexpr bool HD = FORM == 1 || FORM == 4;  // a decay and an input scale per head and token
    const int a_words = CH ? RC * Dk : (HD ? 2 * RC : 0);
    const int buf_words = 2 * RC * Dk + a_words + RC * JB;
    const int g = h / heads_per_group;
    float* S_mem = state + slots[seq] * state_stride + state_off + ((size_t)h * Dv + (live ? j : 0)) * Dk;
    // VEC (Dk == 8 IP): a thread owns channels 4 ipart .. 4 ipart + 3 and the same four in the upper half, read as
    // two 16-byte words per operand and token (neighbouring lanes read neighbouring words: no bank conflicts);
    // otherwise channels ipart, ipart + IP, .. one word at a time
    const int half = Dk >> 1;
    auto channel = [&](int r) { return VEC ? (r < 4 ? 0 : half) + ipart * 4 + (r & 3) : ipart + r * IP; };
    float S[RS], c1[RS];
#pragma unroll
    for (int r = 0; r < RS; ++r) {
        const int i = channel(r);
        const bool on = i < Dk;
        S[r] = (on && live) ? S_mem[i] : 0.f;
        if (FORM == 0) c1[r] = on ? p1[(size_t)h * Dk + i] : 0.f;
    }
    const float head_skip = (FORM == 1 && p2 != nullptr) ? p2[h] : 0.f;
    const float head_decay = FORM == 3 ? p0[h] : 0.f;
    const float* qp = q + (size_t)g * Dk;
    const float* kp = k + (size_t)g * Dk;
    const float* pp = CH ? pre + (size_t)h * Dk : (HD ? pre + h : nullptr);
    const int Dvin = FORM == 4 ? Dv - 1 : Dv;  // value columns that v holds
    const float* vp = v + (size_t)h * Dvin + j0;
    const int nv = min(JB, Dvin - j0);
    auto fetch = [&](int t0, float* buf) {  // raw operands of tokens t0 .. t0+RC-1 (those below `end`)
        const int n = min(RC, end - t0);
        float* qs = buf;
        float* ks = buf + RC * Dk;
        float* as = buf + 2 * RC * Dk;
        float* vs = as + a_words;
        if (wide) {  // rows of whole 16-byte pieces at 16-byte addresses
            const int pieces = Dk >> 2;
            const int shift = VEC ? 31 - __clz(pieces) : 0;  // (VEC: Dk = 8 * 2^n, so a power of two)
            for (int idx = tid; idx < n * pieces; idx += blockDim.x) {
                const int t = VEC ? idx >> shift : idx / pieces, i = (idx - t * pieces) << 2;
                cp_async16f(qs + t * Dk + i, qp + (size_t)(t0 + t) * ldq + i);
                cp_async16f(ks + t * Dk + i, kp + (size_t)(t0 + t) * ldk + i);
                if (CH) cp_async16f(as + t * Dk + i, pp + (size_t)(t0 + t) * ldp + i);
            }
        } else {
            for (int idx = tid; idx < n * Dk; idx += blockDim.x) {
                const int t = idx / Dk, i = idx - t * Dk;
                cp_async4(qs + idx, qp + (size_t)(t0 + t) * ldq + i);
                cp_async4(ks + idx, kp + (size_t)(t0 + t) * ldk + i);
                if (CH) cp_async4(as + idx, pp + (size_t)(t0 + t) * ldp + i);
            }
        }
        if (HD)
            for (int t = tid; t < 2 * n; t += blockDim.x) {  // a and dt of the head
                const int tok = t >> 1, second = t & 1;
                cp_async4(as + second * RC + tok, pp + (size_t)(t0 + tok) * ldp + second * H);
            }
        for (int idx = tid; idx < n * nv; idx += blockDim.x) {
            const int t = idx / nv, c = idx - t * nv;
            cp_async4(vs + t * JB + c, vp + (size_t)(t0 + t) * ldv + c);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(start, rs_smem);
    int which = 0;
    for (int t0 = start; t0 < end; t0 += RC, which ^= 1) {
        const int n = min(RC, end - t0);
        float* buf = rs_smem + which * buf_words;
        float* qs = buf;
        float* ks = buf + RC * Dk;
        float* as = buf + 2 * RC * Dk;
        float* vs = as + a_words;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // this chunk has landed; everyone has left the other buffer
        if (t0 + RC < end) fetch(t0 + RC, rs_smem + (which ^ 1) * buf_words);
        float part[RC];
#pragma unroll
        for (int t = 0; t < RC; ++t) {
            part[t] = 0.f;
            if (t < n) {
                const float vraw = live ? ((FORM == 4 && j == Dv - 1) ? 1.f : vs[t * JB + jl]) : 0.f;
                const float a1 = HD ? as[t] : head_decay;
                const float vc = HD ? vraw * as[RC + t] : vraw;  // the step size scales the update
                float sum = 0.f;
                if (VEC) {
                    const int at = t * Dk + ipart * 4, up = at + half;
                    float kc[RS], qc[RS], ac[RS];
                    *(float4*)&kc[0] = *(const float4*)(ks + at);
                    *(float4*)&kc[4] = *(const float4*)(ks + up);
                    *(float4*)&qc[0] = *(const float4*)(qs + at);
                    *(float4*)&qc[4] = *(const float4*)(qs + up);
                    if (CH) {
                        *(float4*)&ac[0] = *(const float4*)(as + at);
                        *(float4*)&ac[4] = *(const float4*)(as + up);
                    }
                    float sum2 = 0.f;  // two chains of four, added at the end: the same order for every token and batch
#pragma unroll
                    for (int r = 0; r < RS; ++r) {
                        const float kv = kc[r] * vc;
                        float& acc_sum = r < 4 ? sum : sum2;
                        if (FORM == 0) {
                            acc_sum = fmaf(qc[r], fmaf(c1[r], kv, S[r]), acc_sum);
                            S[r] = fmaf(ac[r], S[r], kv);
                        } else {
                            S[r] = fmaf(CH ? ac[r] : a1, S[r], kv);
                            acc_sum = fmaf(qc[r], S[r], acc_sum);
                        }
                    }
                    sum += sum2;
                } else {
#pragma unroll
                    for (int r = 0; r < RS; ++r) {
                        const int i = ipart + r * IP;
                        if (i < Dk) {
                            const float kv = ks[t * Dk + i] * vc, qc = qs[t * Dk + i];
                            if (FORM == 0) {
                                sum = fmaf(qc, fmaf(c1[r], kv, S[r]), sum);
                                S[r] = fmaf(as[t * Dk + i], S[r], kv);
                            } else {
                                S[r] = fmaf(CH ? as[t * Dk + i] : a1, S[r], kv);
                                sum = fmaf(qc, S[r], sum);
                            }
                        }
                    }
                }
                part[t] = sum;
            }
        }
#pragma unroll
        for (int t = 0; t < RC; ++t)
            for (int o = 1; o < IP; o <<= 1) part[t] += __shfl_xor_sync(0xffffffffu, part[t], o);
        if (live && ipart == 0) {
#pragma unroll
            for (int t = 0; t < RC; ++t)
                if (t < n)
                    out[(size_t)(t0 + t) * ldo + (size_t)h * Dv + j] =
                        FORM == 1 ? fmaf(head_skip, vs[t * JB + jl], part[t]) : (FORM >= 2 ? part[t] * q_scale : part[t]);
        }
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < RS; ++r) {
            const int i = channel(r);
            if (i < Dk) S_mem[i] = S[r];
        }
    }
}

// pre: the coefficients that cw_recurrence_coefficients made (form 0: a [N, H*Dk]; form 1: [a | dt] [N, 2H]).
extern "C" int cw_recurrence_scan(int form, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                                  const float* pre, int ldp, const float* p0, const float* p1, const float* p2,
                                  float* state, long long state_stride, long long state_off, const long long* slots,
                                  const int* tok_seq, const int* q_start, int S, int H, int Dk, int Dv, int heads_per_group, float* out, int ldo,
                                  float q_scale, cudaStream_t stream) {
    if (S == 0) return CW_OK;
    if (S < 0 || H <= 0 || Dk <= 0 || Dv <= 0 || heads_per_group <= 0 || H % heads_per_group) return CW_ERR_BAD_SIZE;
    if (Dk > 32 * RS || H > 65535) return CW_ERR_UNSUPPORTED;
    int IP = 1;
    while (IP * RS < Dk) IP *= 2;
    int threads = 256;  // more value columns per block share the staged q and k; fewer when a head has few columns
    while (threads > 32 && threads / IP >= 2 * Dv) threads /= 2;
    const int JB = threads / IP;
    dim3 grid(S, H, (Dv + JB - 1) / JB);
    if (form < 0 || form > 4) return CW_ERR_UNSUPPORTED;
    if (form == 4 && Dv < 2) return CW_ERR_BAD_SIZE;
    const bool ch = form == 0 || form == 2;  // coefficients per key channel
    if ((form != 3 && pre == nullptr) || (form == 3 && p0 == nullptr)) return CW_ERR_BAD_SIZE;
    const int wide = Dk % 4 == 0 && ldq % 4 == 0 && ldk % 4 == 0 && (!ch || ldp % 4 == 0) && ((uintptr_t)q & 15) == 0 &&
                     ((uintptr_t)k & 15) == 0 && (!ch || ((uintptr_t)pre & 15) == 0);
    const size_t smem = 2 * sizeof(float) * (size_t)(2 * RC * Dk + (ch ? RC * Dk : (form == 1 || form == 4 ? 2 * RC : 0)) + RC * JB);
    const bool vec = wide && Dk == IP * RS;
    const int which = form * 2 + (vec ? 1 : 0);
    static size_t allowed[10] = {48 << 10, 48 << 10, 48 << 10, 48 << 10, 48 << 10, 48 << 10, 48 << 10, 48 << 10, 48 << 10, 48 << 10};
    using Kernel = void (*)(const float*, int, const float*, int, const float*, int, const float*, int, const float*, const float*,
                            const float*, float*, long long, long long, const long long*, const int*, const int*, int, int, int, int, int, int,
                            float*, int, float);
    const Kernel kernels[10] = {recurrence_scan_kernel<0, false>, recurrence_scan_kernel<0, true>, recurrence_scan_kernel<1, false>,
                                recurrence_scan_kernel<1, true>, recurrence_scan_kernel<2, false>, recurrence_scan_kernel<2, true>,
                                recurrence_scan_kernel<3, false>, recurrence_scan_kernel<3, true>, recurrence_scan_kernel<4, false>,
                                recurrence_scan_kernel<4, true>};
    if (smem > allowed[which]) {
        const cudaError_t e = cudaFuncSetAttribute(kernels[which], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed[which] = smem;
    }
    return cw_launch_ordered(kernels[which], grid, dim3(threads), smem, stream, q, ldq, k, ldk, v, ldv, pre, ldp, p0, p1, p2, state,
                     state_stride, state_off, slots, tok_seq, q_start, Dk, Dv, heads_per_group, IP, wide, H, out, ldo, q_scale);
}

// Decays of a gated linear-attention layer from the pre-activations of its decay product, in place (float32):
//   a[t, c] = sigmoid(pre[t, c])^(1/tau) = exp(log_sigmoid(pre[t, c]) / tau)
__global__ void __launch_bounds__(256)
sigmoid_power_decay_kernel(float* __restrict__ pre, int ldp, int N, int C, float inv_tau) {
    pdl_wait();
    const long long total = (long long)N * C;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / C), c = (int)(idx - (long long)t * C);
        float* at = pre + (size_t)t * ldp + c;
        const float z = *at;
        const float log_sigmoid = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
        *at = expf(log_sigmoid * inv_tau);
    }
}

extern "C" int cw_sigmoid_power_decay(float* pre, int ldp, int N, int C, float inv_tau, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || C <= 0 || ldp < C) return CW_ERR_BAD_SIZE;
    const long long total = (long long)N * C;
    const int blocks = (int)min((long long)148 * 8, (total + 255) / 256);
    return cw_launch_ordered(sigmoid_power_decay_kernel, dim3(blocks), dim3(256), 0, stream, pre, ldp, N, C, inv_tau);
}

// ---- forget gates with a lower bound ---------------------------------------------------------------------
// On rows [q (C) | z (C) | ..] of a product's float32 output: q <- silu(q);  f = lower + (1 - lower) sigmoid(z + bias) replaces
// z (the decay of a channel of the state), and 1 - f goes to `take` [N, C] (what the channel takes of the new value).
__global__ void __launch_bounds__(256)
bounded_forget_kernel(float* __restrict__ x, int ld, const float* __restrict__ bias, const float* __restrict__ lower,
                      float* __restrict__ take, int N, int C) {
    pdl_wait();
    const long long total = (long long)N * C;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / C), c = (int)(i - (long long)t * C);
        float* row = x + (size_t)t * ld;
        const float q = row[c];
        row[c] = q / (1.f + expf(-q));
        const float z = row[C + c] + (bias != nullptr ? bias[c] : 0.f);
        const float l = lower[c];
        const float f = fmaf(1.f - l, 1.f / (1.f + expf(-z)), l);
        row[C + c] = f;
        take[i] = 1.f - f;
    }
}

extern "C" int cw_bounded_forget(float* x, int ld, const float* bias, const float* lower, float* take, int N, int C,
                                 cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || C <= 0 || ld < 2 * C || lower == nullptr || take == nullptr) return CW_ERR_BAD_SIZE;
    const long long total = (long long)N * C;
    const int blocks = (int)min((long long)148 * 8, (total + 255) / 256);
    return cw_launch_ordered(bounded_forget_kernel, dim3(blocks), dim3(256), 0, stream, x, ld, bias, lower, take, N, C);
}

// ---- gated norm in parts ----------------------------------------------------------------------------
// y [N, C] float32, gate z [N, ldz] float32.  mode bit 0 (gate first): u = y gate(z), out = u / rms_part(u) * weight.
// Otherwise: out = y / rms_part(y) * weight * gate(z).  mode bit 1: gate = sigmoid (else silu).  mode bit 2: every
// part uses the same weight of one part's width.  mode bit 3: no gate at all (z may be null).  A block per (row, part);
// sums in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ z, int ldz, const float* __restrict__ weight,
                        T* __restrict__ out, int C, int parts, float eps, int mode) {
    __shared__ float scratch[33];
    pdl_wait();
    const bool ungated = mode & 8;
    const int gate_first = ungated ? 0 : (mode & 1);
    const bool plain_sigmoid = mode & 2;
    const int row = blockIdx.x, p = blockIdx.y;
    const int width = C / parts;
    const float* yr = y + (size_t)row * C + (size_t)p * width;
    const float* zr = z + (size_t)row * ldz + (size_t)p * width;
    const float* wr = weight + ((mode & 4) ? 0 : (size_t)p * width);
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float u = yr[c];
        if (gate_first) {
            const float g = zr[c];
            u *= (plain_sigmoid ? 1.f : g) / (1.f + expf(-g));
        }
        ss = fmaf(u, u, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float g = ungated ? 0.f : zr[c];
        const float sg = ungated ? 1.f : (plain_sigmoid ? 1.f : g) / (1.f + expf(-g));
        const float u = gate_first ? yr[c] * sg : yr[c];
        float r = u * inv * wr[c];
        if (!gate_first) r *= sg;
        out[(size_t)row * C + (size_t)p * width + c] = from_f<T>(r);
    }
}

extern "C" int cw_gated_group_norm(const float* y, const float* z, int ldz, const float* weight, void* out, int N, int C,
                                   int parts, float eps, int mode, int dtype, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || C <= 0 || parts <= 0 || C % parts || parts > 65535) return CW_ERR_BAD_SIZE;
    if (!(mode & 8) && (z == nullptr || ldz < C)) return CW_ERR_BAD_SIZE;
    const int width = C / parts;
    int threads = 32;
    while (threads < 256 && threads * 4 < width) threads *= 2;
    dim3 grid(N, parts);
    if (dtype == 0)
        return cw_launch_ordered(gated_group_norm_kernel<float>, grid, dim3(threads), 0, stream, y, z, ldz, weight, (float*)out, C, parts,
                         eps, mode);
    if (dtype == 1)
        return cw_launch_ordered(gated_group_norm_kernel<bf16>, grid, dim3(threads), 0, stream, y, z, ldz, weight, (bf16*)out, C, parts,
                         eps, mode);
    return CW_ERR_BAD_DTYPE;
}

// ---- activations in place -----------------------------------------------------------------------------
__device__ __forceinline__ float activation_of(int kind, float z) {
    if (kind == 0) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    if (kind == 1) return tanhf(z);
    const float s = 1.f / (1.f + expf(-z));
    return kind == 2 ? z * s : s;  // silu, sigmoid
}

template <typename T>
__global__ void __launch_bounds__(256) activation_kernel(T* __restrict__ x, long long n, int kind) {
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = from_f<T>(activation_of(kind, to_f(x[i])));
}

// the same on the first C columns of rows that are ld apart
template <typename T>
__global__ void __launch_bounds__(256) activation_cols_kernel(T* __restrict__ x, int ld, int N, int C, int kind) {
    pdl_wait();
    const long long total = (long long)N * C;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / C), c = (int)(i - (long long)t * C);
        T* at = x + (size_t)t * ld + c;
        *at = from_f<T>(activation_of(kind, to_f(*at)));
    }
}

extern "C" int cw_activation_cols(void* x, int ld, int N, int C, int kind, int dtype, cudaStream_t stream) {
    if (N == 0 || C == 0) return CW_OK;
    if (N < 0 || C < 0 || ld < C || kind < 0 || kind > 3) return CW_ERR_BAD_SIZE;
    const long long total = (long long)N * C;
    const int blocks = (int)min((long long)148 * 8, (total + 255) / 256);
    if (dtype == 0) return cw_launch_ordered(activation_cols_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, ld, N, C, kind);
    if (dtype == 1) return cw_launch_ordered(activation_cols_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)x, ld, N, C, kind);
    return CW_ERR_BAD_DTYPE;
}

extern "C" int cw_activation(void* x, long long n, int kind, int dtype, cudaStream_t stream) {
    if (n == 0) return CW_OK;
    if (n < 0 || kind < 0 || kind > 3) return CW_ERR_BAD_SIZE;
    const int blocks = (int)min((long long)148 * 8, (n + 255) / 256);
    if (dtype == 0) return cw_launch_ordered(activation_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, n, kind);
    if (dtype == 1) return cw_launch_ordered(activation_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)x, n, kind);
    return CW_ERR_BAD_DTYPE;
}

CW_TRACE_TU(recurrence)
