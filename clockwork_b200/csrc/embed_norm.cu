// Embedding gather and fused residual-add + RMSNorm.
//
// Reference formulas: clockwork/engine/model.py:200 (embedding), :44-49 (RMSNorm: float32
// statistics, x * rsqrt(mean(x^2) + eps), then the weight), :150 and :154 (residual sums).
// The residual stream is float32 in both run precisions; the normed output has the run's
// activation type.
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table,
                             const int* __restrict__ ids, int H, int V, float scale, int* status) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    const int id = ids[row];
    float* o = out + (size_t)row * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) cw_report(status, CW_ST_TOKEN_RANGE, row, id);
        for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = 0.f;
        return;
    }
    const T* src = table + (size_t)id * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = to_f(src[c]) * scale;  // (scale 1: the row as it is)
}

extern "C" int cw_embed(float* out, const void* table, const int* ids, int N, int H, int V,
                        int dtype, float scale, int* status, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || H <= 0 || V <= 0) return CW_ERR_BAD_SIZE;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == 0)
        return cw_launch(embed_kernel<float>, dim3(N), dim3(threads), 0, stream, 1, out, (const float*)table, ids, H, V, scale, status);
    if (dtype == 1)
        return cw_launch(embed_kernel<bf16>, dim3(N), dim3(threads), 0, stream, 1, out, (const bf16*)table, ids, H, V, scale, status);
    return CW_ERR_BAD_DTYPE;
}

// resid[row] (+= delta[row]); out[r] = weight * (x * rsqrt(mean(x^2)+eps)).
// With `rows` given, output row r is computed from residual row rows[r] (no add is done).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int num_resid_rows, float eps,
                                   int H, int* status) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    int src_row = r;
    if (rows != nullptr) {
        src_row = rows[r];
        if (src_row < 0 || src_row >= num_resid_rows) {
            if (threadIdx.x == 0) cw_report(status, CW_ST_ROW_RANGE, r, src_row);
            for (int c = threadIdx.x; c < H; c += blockDim.x) out[(size_t)r * H + c] = from_f<T>(0.f);
            return;
        }
    }
    float* x = resid + (size_t)src_row * H;
    const T* d = delta ? delta + (size_t)src_row * H : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = x[c];
        if (d) {
            v += to_f(d[c]);
            x[c] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = from_f<T>(weight[c] * (x[c] * inv));
}

// The same for many rows (prompt portions): one warp per row, the row held in registers between the
// sum of squares and the scaling, 16-byte accesses, no block-level synchronisation.  H must be a
// multiple of 4 and at most 128 * NV.
template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <>
struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x), b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 r;
        r.x = *reinterpret_cast<const uint32_t*>(&a);
        r.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

template <typename T, int NV>
__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ weight,
                        T* __restrict__ out, int num_rows, float eps, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= num_rows) return;
    float* x = resid + (size_t)r * H;
    const T* d = delta ? delta + (size_t)r * H : nullptr;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        if (c < H) {
            v[i] = Vec4<float>::load(x + c);
            if (d) {
                const float4 dv = Vec4<T>::load(d + c);
                v[i].x += dv.x; v[i].y += dv.y; v[i].z += dv.z; v[i].w += dv.w;
                Vec4<float>::store(x + c, v[i]);
            }
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        if (c < H) {
            const float4 w = Vec4<float>::load(weight + c);
            Vec4<T>::store(o + c, make_float4(w.x * (v[i].x * inv), w.y * (v[i].y * inv), w.z * (v[i].z * inv), w.w * (v[i].w * inv)));
        }
    }
}

template <typename T>
static int launch_rmsnorm_warp(float* resid, const T* delta, const float* weight, T* out, int rows, int H, float eps,
                               cudaStream_t stream) {
    const int warps = 8;
    const dim3 grid((rows + warps - 1) / warps), block(warps * 32);
    const int nv = (H + 127) / 128;
#define CW_NV(n) \
    if (nv <= n) return cw_launch(add_rmsnorm_warp_kernel<T, n>, grid, block, 0, stream, 1, resid, delta, weight, out, rows, eps, H);
    CW_NV(4) CW_NV(8) CW_NV(12) CW_NV(16) CW_NV(24) CW_NV(32)
#undef CW_NV
    return CW_ERR_UNSUPPORTED;
}

extern "C" int cw_add_rmsnorm(float* resid, const void* delta, const float* weight, void* out,
                              const int* rows, int num_out_rows, int num_resid_rows, int H,
                              float eps, int dtype, int* status, cudaStream_t stream) {
    if (num_out_rows == 0) return CW_OK;
    if (num_out_rows < 0 || H <= 0) return CW_ERR_BAD_SIZE;
    if (rows != nullptr && delta != nullptr) return CW_ERR_UNSUPPORTED;
    // many rows: a warp per row; few rows (decode): a block per row, for the latency of the one row
    const bool aligned = H % 4 == 0 && H <= 4096 && ((uintptr_t)resid & 15) == 0 && ((uintptr_t)weight & 15) == 0 &&
                         ((uintptr_t)out & 15) == 0 && ((uintptr_t)delta & 15) == 0;
    if (rows == nullptr && num_out_rows >= 256 && aligned) {
        if (dtype == 0)
            return launch_rmsnorm_warp<float>(resid, (const float*)delta, weight, (float*)out, num_out_rows, H, eps, stream);
        if (dtype == 1)
            return launch_rmsnorm_warp<bf16>(resid, (const bf16*)delta, weight, (bf16*)out, num_out_rows, H, eps, stream);
        return CW_ERR_BAD_DTYPE;
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (dtype == 0)
        return cw_launch(add_rmsnorm_kernel<float>, dim3(num_out_rows), dim3(threads), 0, stream, 1, resid,
                         (const float*)delta, weight, (float*)out, rows, num_resid_rows, eps, H, status);
    if (dtype == 1)
        return cw_launch(add_rmsnorm_kernel<bf16>, dim3(num_out_rows), dim3(threads), 0, stream, 1, resid,
                         (const bf16*)delta, weight, (bf16*)out, rows, num_resid_rows, eps, H, status);
    return CW_ERR_BAD_DTYPE;
}

// resid[r] += parts[0][r] + parts[1][r] + .. (in this order: the splits of a product over K that were
// kept apart), then, with `out`, out[r] = resid[r] normalised as above.  A warp per row, the row in
// registers between the two passes.
template <typename T, int NV>
__global__ void __launch_bounds__(256)
add_parts_rmsnorm_kernel(float* __restrict__ resid, const float* __restrict__ parts, int num_parts, size_t part_stride,
                         const float* __restrict__ weight, T* __restrict__ out, int num_rows, float eps, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= num_rows) return;
    float* x = resid + (size_t)r * H;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        if (c < H) v[i] = Vec4<float>::load(x + c);
    }
    for (int k = 0; k < num_parts; ++k) {
        const float* d = parts + k * part_stride + (size_t)r * H;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = (i * 32 + lane) * 4;
            if (c < H) {
                const float4 dv = Vec4<float>::load(d + c);
                v[i].x += dv.x; v[i].y += dv.y; v[i].z += dv.z; v[i].w += dv.w;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        if (c < H) {
            Vec4<float>::store(x + c, v[i]);
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    if (out == nullptr) return;
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        if (c < H) {
            const float4 w = Vec4<float>::load(weight + c);
            Vec4<T>::store(o + c, make_float4(w.x * (v[i].x * inv), w.y * (v[i].y * inv), w.z * (v[i].z * inv), w.w * (v[i].w * inv)));
        }
    }
}

template <typename T>
static int launch_add_parts(float* resid, const float* parts, int num_parts, size_t part_stride, const float* weight, T* out,
                            int rows, int H, float eps, cudaStream_t stream) {
    const int warps = 8;
    const dim3 grid((rows + warps - 1) / warps), block(warps * 32);
    const int nv = (H + 127) / 128;
#define CW_NV(n) \
    if (nv <= n) return cw_launch(add_parts_rmsnorm_kernel<T, n>, grid, block, 0, stream, 1, resid, parts, num_parts, part_stride, weight, out, rows, eps, H);
    CW_NV(4) CW_NV(8) CW_NV(12) CW_NV(16) CW_NV(24) CW_NV(32)
#undef CW_NV
    return CW_ERR_UNSUPPORTED;
}

// parts: float32 [num_parts][part_rows][H] (part_rows >= rows); out null: only the sum.  H a multiple of 4,
// at most 4096; 16-byte aligned pointers; CW_ERR_UNSUPPORTED otherwise.
extern "C" int cw_add_parts_rmsnorm(float* resid, const float* parts, int num_parts, int part_rows, const float* weight,
                                    void* out, int rows, int H, float eps, int dtype, cudaStream_t stream) {
    if (rows == 0) return CW_OK;
    if (rows < 0 || H <= 0 || num_parts < 1 || part_rows < rows) return CW_ERR_BAD_SIZE;
    if (H % 4 != 0 || H > 4096 || ((uintptr_t)resid & 15) || ((uintptr_t)parts & 15) || ((uintptr_t)weight & 15) ||
        ((uintptr_t)out & 15))
        return CW_ERR_UNSUPPORTED;
    const size_t stride = (size_t)part_rows * H;
    if (out == nullptr || dtype == 0)
        return launch_add_parts<float>(resid, parts, num_parts, stride, weight, (float*)out, rows, H, eps, stream);
    if (dtype == 1) return launch_add_parts<bf16>(resid, parts, num_parts, stride, weight, (bf16*)out, rows, H, eps, stream);
    return CW_ERR_BAD_DTYPE;
}

// out = silu(gate) * up, gate and up being the two halves of each row of `gate_up` [N, 2*I]
// (clockwork/engine/model.py:62-63).  Used where the product is not fused into the GEMM.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I,
                                size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t row = i / I, col = i % I;
    const float g = to_f(gate_up[row * 2 * I + col]);
    const float u = to_f(gate_up[row * 2 * I + I + col]);
    out[i] = from_f<T>(g / (1.0f + expf(-g)) * u);
}

extern "C" int cw_silu_mul(const void* gate_up, void* out, int N, int I, int dtype,
                           cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || I <= 0) return CW_ERR_BAD_SIZE;
    const size_t total = (size_t)N * I;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == 0)
        silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, I, total);
    else if (dtype == 1)
        silu_mul_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, I, total);
    else
        return CW_ERR_BAD_DTYPE;
    return CW_LAUNCH_CHECK();
}

// resid += delta (float32 += T); used where a part returns a delta that no norm follows.
template <typename T>
__global__ void add_to_residual_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                       size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) resid[i] += to_f(delta[i]);
}

extern "C" int cw_add_to_residual(float* resid, const void* delta, int N, int H, int dtype,
                                  cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || H <= 0) return CW_ERR_BAD_SIZE;
    const size_t total = (size_t)N * H;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0)
        add_to_residual_kernel<float><<<blocks, 256, 0, stream>>>(resid, (const float*)delta, total);
    else if (dtype == 1)
        add_to_residual_kernel<bf16><<<blocks, 256, 0, stream>>>(resid, (const bf16*)delta, total);
    else
        return CW_ERR_BAD_DTYPE;
    return CW_LAUNCH_CHECK();
}

// ---- an embedding's scale and absolute positions ------------------------------------------------------
// x[row, c] <- x[row, c] * scale + (c even ? sin : cos)(position[row] * inv_freq[c / 2]): the sinusoidal
// position vector of width W added to the (scaled) embedding rows.  Angles in float32.
__global__ void __launch_bounds__(256)
scale_add_sinusoid_kernel(float* __restrict__ x, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                          float scale, int W) {
    pdl_wait();
    const int row = blockIdx.x;
    const float p = (float)positions[row];
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float angle = p * inv_freq[c >> 1];
        const float pe = (c & 1) ? cosf(angle) : sinf(angle);
        x[(size_t)row * W + c] = fmaf(x[(size_t)row * W + c], scale, pe);
    }
}

extern "C" int cw_scale_add_sinusoid(float* x, const int* positions, const float* inv_freq, float scale, int N, int W,
                                     cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || W <= 0) return CW_ERR_BAD_SIZE;
    return cw_launch_ordered(scale_add_sinusoid_kernel, dim3(N), dim3(256), 0, stream, x, positions, inv_freq, scale, W);
}

// ---- two contributions, each normed over the width, into the residual ---------------------------------
// resid[row] += factor * (a[row] / rms(a[row]) * wa + b[row] / rms(b[row]) * wb), everything float32.
__global__ void __launch_bounds__(256)
pair_rmsnorm_add_kernel(float* __restrict__ resid, const float* __restrict__ a, const float* __restrict__ b,
                        const float* __restrict__ wa, const float* __restrict__ wb, float eps, float factor, int W) {
    __shared__ float scratch[33];
    pdl_wait();
    const size_t at = (size_t)blockIdx.x * W;
    float sa = 0.f, sb = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float u = a[at + c], v = b[at + c];
        sa = fmaf(u, u, sa);
        sb = fmaf(v, v, sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ia = 1.0f / sqrtf(sa / (float)W + eps), ib = 1.0f / sqrtf(sb / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x)
        resid[at + c] += factor * (a[at + c] * ia * wa[c] + b[at + c] * ib * wb[c]);
}

extern "C" int cw_pair_rmsnorm_add(float* resid, const float* a, const float* b, const float* wa, const float* wb, float eps,
                                   float factor, int N, int W, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || W <= 0) return CW_ERR_BAD_SIZE;
    return cw_launch_ordered(pair_rmsnorm_add_kernel, dim3(N), dim3(256), 0, stream, resid, a, b, wa, wb, eps, factor, W);
}

// ---- a weighted sum of contributions, normed over the width, into the residual ------------------------
// y = ca a (+ cb b);  resid[row] += y / sqrt(mean(y^2) + eps) * w, everything float32 (b may be null).
__global__ void __launch_bounds__(256)
sum_rmsnorm_add_kernel(float* __restrict__ resid, const float* __restrict__ a, const float* __restrict__ b, float ca, float cb,
                       const float* __restrict__ w, float eps, int W) {
    __shared__ float scratch[33];
    pdl_wait();
    const size_t at = (size_t)blockIdx.x * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float y = b != nullptr ? fmaf(cb, b[at + c], ca * a[at + c]) : ca * a[at + c];
        ss = fmaf(y, y, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float y = b != nullptr ? fmaf(cb, b[at + c], ca * a[at + c]) : ca * a[at + c];
        resid[at + c] += y * inv * w[c];
    }
}

extern "C" int cw_sum_rmsnorm_add(float* resid, const float* a, const float* b, float ca, float cb, const float* w, float eps,
                                  int N, int W, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || W <= 0 || a == nullptr) return CW_ERR_BAD_SIZE;
    int threads = 64;
    while (threads < 256 && threads * 4 < W) threads *= 2;
    return cw_launch_ordered(sum_rmsnorm_add_kernel, dim3(N), dim3(threads), 0, stream, resid, a, b, ca, cb, w, eps, W);
}

// ---- logits bent towards a bound ------------------------------------------------------------------------
// x <- cap tanh(x / cap), in place, float32.
__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ x, long long n, float cap) {
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

extern "C" int cw_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n == 0) return CW_OK;
    if (n < 0 || !(cap > 0.f)) return CW_ERR_BAD_SIZE;
    const int blocks = (int)min((long long)148 * 8, (n + 255) / 256);
    return cw_launch_ordered(softcap_kernel, dim3(blocks), dim3(256), 0, stream, x, n, cap);
}

// ---- a second table read by a hash of (previous token, token) -------------------------------------------
// x[n] += table[row], row = (previous * mul_prev + token * mul_cur) mod buckets; a request's first token reads row
// `buckets` (the table has buckets + 1 rows).  The token before a portion's first one is what the step before left in
// the request's state (one int32 per request: state[slots[s] * stride]); keep_last_token_kernel, launched after this
// one, leaves the portion's last token there.  Rows of no request (tok_seq < 0) are left alone.
template <typename T>
__global__ void __launch_bounds__(256)
pair_embed_add_kernel(float* __restrict__ x, const T* __restrict__ table, const int* __restrict__ ids,
                      const int* __restrict__ positions, const int* __restrict__ tok_seq, const int* __restrict__ q_start,
                      const int* __restrict__ state, long long stride, const long long* __restrict__ slots, int buckets,
                      long long mul_prev, long long mul_cur, int W, int V, int* __restrict__ status) {
    pdl_wait();
    const int n = blockIdx.x;
    const int seq = tok_seq[n];
    if (seq < 0) return;
    const int tok = ids[n];
    int prev = -1;
    if (n > q_start[seq])
        prev = ids[n - 1];
    else if (positions[n] > 0)
        prev = state[slots[seq] * stride];
    if (tok < 0 || tok >= V || prev >= V) {
        if (threadIdx.x == 0) cw_report(status, CW_ST_TOKEN_RANGE, n, tok);
        return;
    }
    long long row = buckets;
    if (prev >= 0) {
        row = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
        if (row < 0) row += buckets;
    }
    const T* from = table + (size_t)row * W;
    float* to = x + (size_t)n * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) to[c] += to_f(from[c]);
}

__global__ void __launch_bounds__(128)
keep_last_token_kernel(const int* __restrict__ ids, const int* __restrict__ tok_seq, const int* __restrict__ q_start,
                       int* __restrict__ state, long long stride, const long long* __restrict__ slots, int S) {
    pdl_wait();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= S) return;
    const int a = q_start[s], b = q_start[s + 1];
    if (b <= a || tok_seq[a] < 0) return;
    state[slots[s] * stride] = ids[b - 1];
}

extern "C" int cw_pair_embed_add(float* x, const void* table, const int* ids, const int* positions, const int* tok_seq,
                                 const int* q_start, int* state, long long stride, const long long* slots, int buckets,
                                 long long mul_prev, long long mul_cur, int N, int S, int W, int V, int dtype, int* status,
                                 cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || S <= 0 || W <= 0 || buckets <= 0 || stride <= 0) return CW_ERR_BAD_SIZE;
    int threads = 64;
    while (threads < 256 && threads * 4 < W) threads *= 2;
    int rc;
    if (dtype == 0)
        rc = cw_launch_ordered(pair_embed_add_kernel<float>, dim3(N), dim3(threads), 0, stream, x, (const float*)table, ids, positions,
                               tok_seq, q_start, (const int*)state, stride, slots, buckets, mul_prev, mul_cur, W, V, status);
    else if (dtype == 1)
        rc = cw_launch_ordered(pair_embed_add_kernel<bf16>, dim3(N), dim3(threads), 0, stream, x, (const bf16*)table, ids, positions,
                               tok_seq, q_start, (const int*)state, stride, slots, buckets, mul_prev, mul_cur, W, V, status);
    else
        return CW_ERR_BAD_DTYPE;
    if (rc != 0) return rc;
    // (after the reader, in stream order: no block reads a token that another has just replaced)
    return cw_launch_ordered(keep_last_token_kernel, dim3((S + 127) / 128), dim3(128), 0, stream, ids, tok_seq, q_start, state, stride,
                             slots, S);
}

// ---- a scaled contribution into the residual, and the norm that reads it -----------------------------------
// y = x + ca a (+ cb b) goes to `sum` (which may be x itself); out = y / sqrt(mean(y^2) + eps) * w.  Everything float32
// but `out`.
template <typename T>
__global__ void __launch_bounds__(256)
axpy_rmsnorm_kernel(const float* x, const float* __restrict__ a, const float* __restrict__ b, float ca, float cb,
                    float* sum, const float* __restrict__ w, T* __restrict__ out, float eps, int W) {
    __shared__ float scratch[33];
    pdl_wait();
    const size_t at = (size_t)blockIdx.x * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float y = fmaf(ca, a[at + c], x[at + c]);
        if (b != nullptr) y = fmaf(cb, b[at + c], y);
        sum[at + c] = y;
        ss = fmaf(y, y, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) out[at + c] = from_f<T>(sum[at + c] * inv * w[c]);  // (the thread's own writes)
}

extern "C" int cw_axpy_rmsnorm(const float* x, const float* a, const float* b, float ca, float cb, float* sum, const float* w,
                               void* out, float eps, int N, int W, int dtype, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || W <= 0 || a == nullptr || x == nullptr || sum == nullptr) return CW_ERR_BAD_SIZE;
    int threads = 64;
    while (threads < 256 && threads * 4 < W) threads *= 2;
    if (dtype == 0)
        return cw_launch_ordered(axpy_rmsnorm_kernel<float>, dim3(N), dim3(threads), 0, stream, x, a, b, ca, cb, sum, w, (float*)out, eps, W);
    if (dtype == 1)
        return cw_launch_ordered(axpy_rmsnorm_kernel<bf16>, dim3(N), dim3(threads), 0, stream, x, a, b, ca, cb, sum, w, (bf16*)out, eps, W);
    return CW_ERR_BAD_DTYPE;
}

// ---- the weighted average over the depth ------------------------------------------------------------------
// history [runs + 1][N][W] holds what the input rows were (plane 0) and what every layer run left (plane r + 1).  This
// kernel finishes run `index - 1`: y = x + ca a (+ cb b) (a may be null: y = x) goes to plane `index`, and what the next
// layer reads is next = sum over j <= index of coef[j] * plane j, in the order of j.  x may be plane `index` itself, and
// `next` may be x when x is no plane.  With a norm weight the rows of `next` are also normed into `normed`.
template <typename T>
__global__ void __launch_bounds__(256)
depth_average_kernel(const float* x, const float* __restrict__ a, const float* __restrict__ b, float ca, float cb,
                     float* history, long long plane, int index, const float* __restrict__ coef, float* next,
                     const float* __restrict__ w, T* __restrict__ normed, float eps, int W) {
    __shared__ float scratch[33];
    pdl_wait();
    const size_t at = (size_t)blockIdx.x * W;
    float ss = 0.f;
    if ((W & 3) == 0 && (plane & 3) == 0) {  // four columns a thread, 16-byte accesses (every pointer is a tensor's start or a plane's)
        for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
            float4 y = *(const float4*)(x + at + c);
            if (a != nullptr) {
                const float4 t = *(const float4*)(a + at + c);
                y.x = fmaf(ca, t.x, y.x); y.y = fmaf(ca, t.y, y.y); y.z = fmaf(ca, t.z, y.z); y.w = fmaf(ca, t.w, y.w);
            }
            if (b != nullptr) {
                const float4 t = *(const float4*)(b + at + c);
                y.x = fmaf(cb, t.x, y.x); y.y = fmaf(cb, t.y, y.y); y.z = fmaf(cb, t.z, y.z); y.w = fmaf(cb, t.w, y.w);
            }
            *(float4*)(history + (size_t)index * plane + at + c) = y;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < index; ++j) {
                const float k = coef[j];
                const float4 t = *(const float4*)(history + (size_t)j * plane + at + c);
                acc.x = fmaf(k, t.x, acc.x); acc.y = fmaf(k, t.y, acc.y); acc.z = fmaf(k, t.z, acc.z); acc.w = fmaf(k, t.w, acc.w);
            }
            const float k = coef[index];
            acc.x = fmaf(k, y.x, acc.x); acc.y = fmaf(k, y.y, acc.y); acc.z = fmaf(k, y.z, acc.z); acc.w = fmaf(k, y.w, acc.w);
            *(float4*)(next + at + c) = acc;
            ss = fmaf(acc.x, acc.x, fmaf(acc.y, acc.y, fmaf(acc.z, acc.z, fmaf(acc.w, acc.w, ss))));
        }
    } else {
        for (int c = threadIdx.x; c < W; c += blockDim.x) {
            float y = x[at + c];
            if (a != nullptr) y = fmaf(ca, a[at + c], y);
            if (b != nullptr) y = fmaf(cb, b[at + c], y);
            history[(size_t)index * plane + at + c] = y;
            float acc = 0.f;
            for (int j = 0; j < index; ++j) acc = fmaf(coef[j], history[(size_t)j * plane + at + c], acc);
            acc = fmaf(coef[index], y, acc);
            next[at + c] = acc;
            ss = fmaf(acc, acc, ss);
        }
    }
    if (w == nullptr) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) normed[at + c] = from_f<T>(next[at + c] * inv * w[c]);
}

extern "C" int cw_depth_average(const float* x, const float* a, const float* b, float ca, float cb, float* history, long long plane,
                                int index, const float* coef, float* next, const float* w, void* normed, float eps, int N, int W,
                                int dtype, cudaStream_t stream) {
    if (N == 0) return CW_OK;
    if (N < 0 || W <= 0 || index < 1 || plane < (long long)N * W || x == nullptr || history == nullptr || coef == nullptr || next == nullptr)
        return CW_ERR_BAD_SIZE;
    if (w != nullptr && normed == nullptr) return CW_ERR_BAD_SIZE;
    int threads = 64;
    while (threads < 256 && threads * 4 < W) threads *= 2;
    if (dtype == 0)
        return cw_launch_ordered(depth_average_kernel<float>, dim3(N), dim3(threads), 0, stream, x, a, b, ca, cb, history, plane, index, coef,
                                 next, w, (float*)normed, eps, W);
    if (dtype == 1)
        return cw_launch_ordered(depth_average_kernel<bf16>, dim3(N), dim3(threads), 0, stream, x, a, b, ca, cb, history, plane, index, coef,
                                 next, w, (bf16*)normed, eps, W);
    return CW_ERR_BAD_DTYPE;
}

static int g_pdl = 1;
extern "C" int cw_pdl_enabled() { return g_pdl; }
extern "C" int cw_set_pdl(int on) { g_pdl = on ? 1 : 0; return CW_OK; }

CW_TRACE_TU(embed_norm)
