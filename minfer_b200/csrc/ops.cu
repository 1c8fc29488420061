// Row-wise and element-wise kernels of the step: embedding lookup, RMSNorm, the fused
// rotary + cache write, SwiGLU, row gather, casts.  All reductions are in float32.
//
// Formulas follow the reference's CPU backend: get_rows src/graph/cpu_backend.rs:249-291,
// rms_norm src/vec_ops.rs:500-522 (x * 1/sqrt(mean(x^2)+eps) * w), rotary
// src/graph/cpu_backend.rs:403-434, KV store src/graph/cpu_backend.rs:118-149, silu
// src/vec_ops.rs:131-146.  Its CUDA versions (src/cuda_kernels.cu:531-668) launch one
// kernel per op and one thread per block for the KV store; here bias, rotation and both
// cache writes are one pass over the projection's output.
#include "common.cuh"

// ------------------------------------------------------------------------------------
// embedding: out[t][:] = table[ids[t]][:] * scale  (float32 out: the residual stream is
// float32; scale is 1 for architectures that do not multiply their embeddings)
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int width, int vocab, float scale,
                             unsigned* __restrict__ status) {
    pdl_prologue();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * width;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, MF_STATUS_BAD_TOKEN);
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const T* row = table + (size_t)id * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = to_f32(row[i]) * scale;
}

extern "C" int mf_embed(const void* table, int table_dtype, const int* ids, float* out,
                        int n_tokens, int width, int vocab, float scale, unsigned* status,
                        cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == MF_DTYPE_F32)
        mf_launch(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, ids, out, width,
                                                             vocab, scale, status);
    else if (table_dtype == MF_DTYPE_BF16)
        mf_launch(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, 
            (const __nv_bfloat16*)table, ids, out, width, vocab, scale, status);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// RMSNorm over rows of the float32 residual stream; optional row gather (rows[r] names the
// input row of output row r).  y = x * rsqrt(mean(x^2) + eps) * w
// ------------------------------------------------------------------------------------
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               const int* __restrict__ rows, TO* __restrict__ y, int width,
                               float eps) {
    pdl_prologue();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * width;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TO* yr = y + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) yr[i] = from_f32<TO>(xr[i] * scale * w[i]);
}

// four neighbouring outputs in one store
template <typename T> struct Pack4;
template <> struct Pack4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    }
};
template <> struct Pack4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 v;
        v.x = *reinterpret_cast<unsigned*>(&lo);
        v.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(p) = v;
    }
};

// the same with float4 accesses and the row kept in registers (one pass over memory), for
// widths that are multiples of 4 up to 16384
template <typename TO>
__global__ void __launch_bounds__(1024)
rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                   const int* __restrict__ rows, TO* __restrict__ y, int width, float eps) {
    // the norm's weights (and the row to take, an input of the step) are fetched while the
    // kernel before this one still runs
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int nv = width >> 2;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * width);
    float4 g[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) g[j] = reinterpret_cast<const float4*>(w)[i];
    }
    pdl_wait();
    float4 row[4];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            const float4 v = xr[i];
            row[j] = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TO* yr = y + (size_t)r * width;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            const float4 v = row[j];
            Pack4<TO>::store(yr + 4 * i, v.x * scale * g[j].x, v.y * scale * g[j].y,
                             v.z * scale * g[j].z, v.w * scale * g[j].w);
        }
    }
}

extern "C" int mf_rmsnorm(const float* x, const float* w, const int* rows, void* y, int out_dtype,
                          int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width % 4 == 0 && width <= 16384 && (out_dtype == MF_DTYPE_F32 || out_dtype == MF_DTYPE_BF16)) {
        // up to four float4 a thread: fewer warps to sum over, more rows on an SM at once
        // (2,048 rows of 3,584: 6.1 us with 256 threads, 13.1 us with 1,024)
        int threads = 32;
        while (threads < 1024 && threads * 16 < width) threads <<= 1;
        if (out_dtype == MF_DTYPE_F32)
            mf_launch(rmsnorm_vec_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, w, rows,
                      (float*)y, width, eps);
        else
            mf_launch(rmsnorm_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, w,
                      rows, (__nv_bfloat16*)y, width, eps);
        return MF_LAUNCH_CHECK();
    }
    // the block size is a function of the width only, so a row's sum never depends on the batch
    int threads = 32;
    while (threads < 512 && threads * 4 < width) threads <<= 1;
    if (out_dtype == MF_DTYPE_F32)
        mf_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, w, rows, (float*)y, width, eps);
    else if (out_dtype == MF_DTYPE_BF16)
        mf_launch(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, w, rows, (__nv_bfloat16*)y,
                                                                      width, eps);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// Residual add + RMSNorm in one pass: h[r] += bias + sum_s partial[s][r] (the K splits of the
// projection before it, added in split order), then y[r] = rmsnorm(h[r]) * w.  Saves the
// separate reduction kernel and one round trip of h.
// ------------------------------------------------------------------------------------
template <typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ partial,
                                   int n_partials, const float* __restrict__ bias,
                                   const float* __restrict__ w, TO* __restrict__ y, int n_rows,
                                   int width, float eps) {
    pdl_prologue();
    extern __shared__ float row_s[];                  // the updated row
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    float* hr = h + (size_t)r * width;
    const size_t plane = (size_t)n_rows * width;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float add = 0.0f;
        for (int s = 0; s < n_partials; ++s) add += partial[s * plane + (size_t)r * width + i];
        if (bias) add += bias[i];
        const float v = hr[i] + add;
        hr[i] = v;
        row_s[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TO* yr = y + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) yr[i] = from_f32<TO>(row_s[i] * scale * w[i]);
}

// the same for widths that are multiples of 4 up to 4 * 4 * 1024: float4 accesses, the row
// kept in registers, all loads of a thread independent of each other
#define ARN_MAXV 4
template <typename TO, int MAXV>
__global__ void __launch_bounds__(1024)
add_rmsnorm_vec_kernel(float* __restrict__ h, const float* __restrict__ partial, int n_partials,
                       const float* __restrict__ bias, const float* __restrict__ w,
                       TO* __restrict__ y, int n_rows, int width, float eps) {
    // the norm's weights are fetched while the kernel before this one still runs
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int nv = width >> 2;                         // float4 per row
    float4* hr = reinterpret_cast<float4*>(h + (size_t)r * width);
    const size_t plane4 = ((size_t)n_rows * width) >> 2;
    const float4* pr = reinterpret_cast<const float4*>(partial) + ((size_t)r * width >> 2);
    float4 g[MAXV];
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) g[j] = reinterpret_cast<const float4*>(w)[i];
    }
    pdl_wait();
    float4 row[MAXV];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            float4 v;
            if (MAXV == 1) v = hr[i];                 // in flight together with the splits
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll (MAXV == 1 ? 10 : 4)
            for (int s = 0; s < n_partials; ++s) {
                const float4 p = pr[s * plane4 + i];
                acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
            }
            if (bias) {
                const float4 b = reinterpret_cast<const float4*>(bias)[i];
                acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
            }
            if (MAXV != 1) v = hr[i];
            v.x += acc.x; v.y += acc.y; v.z += acc.z; v.w += acc.w;
            hr[i] = v;
            row[j] = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TO* yr = y + (size_t)r * width;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            const float4 v = row[j];
            Pack4<TO>::store(yr + 4 * i, v.x * scale * g[j].x, v.y * scale * g[j].y,
                             v.z * scale * g[j].z, v.w * scale * g[j].w);
        }
    }
}

extern "C" int mf_add_rmsnorm(float* h, const float* partial, int n_partials, const float* bias,
                              const float* w, void* y, int out_dtype, int n_rows, int width,
                              float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_partials < 0 || (n_partials > 0 && partial == nullptr)) return MF_ERR_ARGUMENT;
    if (width % 4 == 0 && width <= 4 * ARN_MAXV * 1024 && (out_dtype == MF_DTYPE_F32 ||
                                                            out_dtype == MF_DTYPE_BF16)) {
        // one thread per float4 where that fits; the block size depends on the width only
        int threads = 32;
        while (threads < 1024 && threads * 4 < width) threads <<= 1;
        if (out_dtype == MF_DTYPE_F32)
            mf_launch(add_rmsnorm_vec_kernel<float, ARN_MAXV>, dim3(n_rows), dim3(threads), 0, stream,
                h, partial, n_partials, bias, w, (float*)y, n_rows, width, eps);
        else if (width <= 4 * 1024)        // one float4 a thread: more splits in flight at once
            mf_launch(add_rmsnorm_vec_kernel<__nv_bfloat16, 1>, dim3(n_rows), dim3(threads), 0, stream,
                h, partial, n_partials, bias, w, (__nv_bfloat16*)y, n_rows, width, eps);
        else
            mf_launch(add_rmsnorm_vec_kernel<__nv_bfloat16, ARN_MAXV>, dim3(n_rows), dim3(threads), 0, stream,
                h, partial, n_partials, bias, w, (__nv_bfloat16*)y, n_rows, width, eps);
        return MF_LAUNCH_CHECK();
    }
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return MF_ERR_UNSUPPORTED;
    int threads = 32;
    while (threads < 512 && threads * 4 < width) threads <<= 1;
    if (out_dtype == MF_DTYPE_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mf_launch(add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, h, partial, n_partials, bias, w,
                                                                    (float*)y, n_rows, width, eps);
    } else if (out_dtype == MF_DTYPE_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mf_launch(add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream, 
            h, partial, n_partials, bias, w, (__nv_bfloat16*)y, n_rows, width, eps);
    } else {
        return MF_ERR_UNSUPPORTED;
    }
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// rotary + cache write.  Input: the fused projection's float32 output qkv[t] =
// [q (n_heads*hd) | k (n_kv*hd) | v (n_kv*hd)], bias already added.  Rotates q and k by
// the token's position (angle pos * inv_freq[i] formed and reduced mod 2 pi in double, its sine
// and cosine in float32), writes
//   q_out[t][h][:]              (activation type)
//   k_out[t][hk][:], v_out[..]  (activation type; the step's own keys and values, which
//                                prefill attention reads; may be null)
//   cache pages                 (if k_cache is not null): position p of batch row b lies in
//                                page page_table[b*table_stride + (p' / 64)], p' = p % ring
//                                for a ring of `ring` positions, else p; inside the page at
//                                [kv_head][p % 64][:].
// A ring holds only the last `ring` positions: a prompt longer than the ring writes just
// those (seq_end[b] is the sequence's length after this step).
// style: 0 = pairs (i, i + R/2) ("NeoX", the reference's NonInterleaved), 1 = pairs
// (2i, 2i+1); R = rotary_dim <= hd, dimensions beyond R pass through; inv_freq null = no
// rotation at all.
// n_partials > 0: `qkv` holds [n_partials][tokens][width] K splits of the projection, which
// are added here in split order together with `bias` (else bias must already be inside).
// ------------------------------------------------------------------------------------
// The angle pos * inv_freq reduced to [0, 2 pi): product and reduction in double (a float32
// product is off by 1e-4 rad at position 2,000 and by 2e-3 rad at 32,000), sine and cosine of
// the small remainder in float32.
__device__ __forceinline__ float rotary_angle(int pos, double inv_freq) {
    const double two_pi = 6.283185307179586476925286766559;
    const double th = (double)pos * inv_freq;
    return (float)(th - two_pi * floor(th / two_pi));
}

template <typename T>
__global__ void rope_kvstore_kernel(const float* __restrict__ qkv, int n_partials, int n_tokens,
                                    const float* __restrict__ bias,
                                    const int* __restrict__ positions,
                                    const int* __restrict__ token_row,
                                    const int* __restrict__ seq_end,
                                    const double* __restrict__ inv_freq, T* __restrict__ q_out,
                                    T* __restrict__ k_out, T* __restrict__ v_out,
                                    T* __restrict__ k_cache, T* __restrict__ v_cache,
                                    const int* __restrict__ page_table, int table_stride, int ring,
                                    int n_heads, int n_kv, int hd, int rotary_dim, int style,
                                    unsigned* __restrict__ status) {
    pdl_prologue();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int b = token_row[t];
    const int half = hd >> 1;
    const int rhalf = rotary_dim >> 1;
    const int n_slots = (n_heads + 2 * n_kv) * half;
    const size_t in_width = (size_t)(n_heads + 2 * n_kv) * hd;
    const float* in = qkv + (size_t)t * in_width;
    const size_t plane = (size_t)n_tokens * in_width;
    // value of element `col` of this token's projection
    auto value = [&](int col) -> float {
        float v = in[col];
        for (int sp = 1; sp < n_partials; ++sp) v += in[sp * plane + col];
        if (bias != nullptr) v += bias[col];
        return v;
    };

    // where this token's keys and values go in the cache
    long long cache_row = -1;     // element offset of [kv_head 0][pos%64][0] in the page, or -1
    if (k_cache != nullptr) {
        bool keep = true;
        int p_eff = pos;
        if (ring > 0) {
            keep = pos >= seq_end[b] - ring;
            p_eff = pos % ring;
        }
        if (keep) {
            const int page = page_table[(size_t)b * table_stride + (p_eff >> 6)];
            if (page < 0) {
                if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, MF_STATUS_BAD_POSITION);
            } else {
                cache_row = ((long long)page * n_kv * MF_PAGE + (pos & (MF_PAGE - 1))) * hd;
            }
        }
    }

    // the token's rotation (cos, sin) per pair, once per block: every head uses the same
    __shared__ float2 cs_table[128];
    if (inv_freq != nullptr) {
        for (int i = threadIdx.x; i < rhalf; i += blockDim.x) {
            float sn, cs;
            sincosf(rotary_angle(pos, inv_freq[i]), &sn, &cs);
            cs_table[i] = make_float2(cs, sn);
        }
    }
    __syncthreads();
    // blockIdx.y spreads a token's pairs over several blocks when there are few tokens
    for (int s = blockIdx.y * blockDim.x + threadIdx.x; s < n_slots; s += gridDim.y * blockDim.x) {
        const int head = s / half;      // 0..n_heads-1: q, then k heads, then v heads
        const int i = s - head * half;
        const int hbase = head * hd;
        int d0, d1;
        float x0, x1;
        const bool is_v = head >= n_heads + n_kv;
        if (!is_v && inv_freq != nullptr && i < rhalf) {
            if (style == 0) { d0 = i; d1 = i + rhalf; } else { d0 = 2 * i; d1 = 2 * i + 1; }
            const float a = value(hbase + d0), c = value(hbase + d1);
            const float cs = cs_table[i].x, sn = cs_table[i].y;
            x0 = a * cs - c * sn;
            x1 = a * sn + c * cs;
        } else {
            // pass-through pair: for rotated heads the dimensions beyond R, else (2i, 2i+1)
            const int j = (!is_v && inv_freq != nullptr) ? rotary_dim + 2 * (i - rhalf) : 2 * i;
            d0 = j; d1 = j + 1;
            x0 = value(hbase + d0);
            x1 = value(hbase + d1);
        }
        const T y0 = from_f32<T>(x0), y1 = from_f32<T>(x1);
        if (head < n_heads) {
            T* o = q_out + ((size_t)t * n_heads + head) * hd;
            o[d0] = y0; o[d1] = y1;
        } else {
            const int hk = is_v ? head - n_heads - n_kv : head - n_heads;
            T* step_out = is_v ? v_out : k_out;
            if (step_out != nullptr) {
                T* o = step_out + ((size_t)t * n_kv + hk) * hd;
                o[d0] = y0; o[d1] = y1;
            }
            if (cache_row >= 0) {
                T* c = (is_v ? v_cache : k_cache) + cache_row + (long long)hk * MF_PAGE * hd;
                c[d0] = y0; c[d1] = y1;
            }
        }
    }
}

// The common case in wide accesses: pairs (i, i + hd/2), the whole head rotated, head sizes
// that are multiples of 8.  A thread takes 4 neighbouring pairs of a q or k head (two float4
// loads per split, two 4-element stores per destination) or 8 elements of a v head.
// SPLIT: the input holds K splits of the projection (decoding: few tokens, every load of a
// thread in flight at once); without it the kernel keeps few registers, so that many CTAs of
// a long prompt share an SM and hide each other's loads.
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(128)
rope_kvstore_vec_kernel(const float* __restrict__ qkv, int n_partials, int n_tokens,
                        const float* __restrict__ bias, const int* __restrict__ positions,
                        const int* __restrict__ token_row, const int* __restrict__ seq_end,
                        const double* __restrict__ inv_freq, T* __restrict__ q_out,
                        T* __restrict__ k_out, T* __restrict__ v_out, T* __restrict__ k_cache,
                        T* __restrict__ v_cache, const int* __restrict__ page_table,
                        int table_stride, int ring, int n_heads, int n_kv, int hd,
                        unsigned* __restrict__ status) {
    // Positions, rows, page tables, inverse frequencies and the bias are the step's inputs
    // (copied to the device before its first kernel) or weights: they are read, and the
    // angles' sines and cosines formed, while the projection before this kernel still runs.
    pdl_launch_dependents();
    __shared__ float2 cs_table[128];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int b = token_row[t];
    const int half = hd >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(rotary_angle(pos, inv_freq[i]), &sn, &cs);
        cs_table[i] = make_float2(cs, sn);
    }
    const size_t in_width = (size_t)(n_heads + 2 * n_kv) * hd;
    const float* in = qkv + (size_t)t * in_width;
    const size_t plane = (size_t)n_tokens * in_width;
    // the sums of two columns at once: all loads of up to 8 splits are issued before the first
    // addition (splits are added in split order, as everywhere)
    auto load_pair = [&](int col_a, int col_c, float4& a, float4& c) {
        a = *reinterpret_cast<const float4*>(in + col_a);
        c = *reinterpret_cast<const float4*>(in + col_c);
        for (int s0 = 1; SPLIT && s0 < n_partials; s0 += 8) {
            float4 pa[8], pc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < n_partials) {
                    pa[j] = *reinterpret_cast<const float4*>(in + (s0 + j) * plane + col_a);
                    pc[j] = *reinterpret_cast<const float4*>(in + (s0 + j) * plane + col_c);
                }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < n_partials) {
                    a.x += pa[j].x; a.y += pa[j].y; a.z += pa[j].z; a.w += pa[j].w;
                    c.x += pc[j].x; c.y += pc[j].y; c.z += pc[j].z; c.w += pc[j].w;
                }
        }
        if (bias != nullptr) {
            const float4 ba = *reinterpret_cast<const float4*>(bias + col_a);
            const float4 bc = *reinterpret_cast<const float4*>(bias + col_c);
            a.x += ba.x; a.y += ba.y; a.z += ba.z; a.w += ba.w;
            c.x += bc.x; c.y += bc.y; c.z += bc.z; c.w += bc.w;
        }
    };
    long long cache_row = -1;
    if (k_cache != nullptr) {
        bool keep = true;
        int p_eff = pos;
        if (ring > 0) {
            keep = pos >= seq_end[b] - ring;
            p_eff = pos % ring;
        }
        if (keep) {
            const int page = page_table[(size_t)b * table_stride + (p_eff >> 6)];
            if (page < 0) {
                if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, MF_STATUS_BAD_POSITION);
            } else {
                cache_row = ((long long)page * n_kv * MF_PAGE + (pos & (MF_PAGE - 1))) * hd;
            }
        }
    }
    __syncthreads();
    pdl_wait();                    // from here on: the projection's sums
    const int upr = half >> 2;                         // units per rotated head
    const int n_rot = (n_heads + n_kv) * upr;
    const int upv = hd >> 3;                           // units per value head
    const int n_units = n_rot + n_kv * upv;
    for (int u = blockIdx.y * blockDim.x + threadIdx.x; u < n_units; u += gridDim.y * blockDim.x) {
        if (u < n_rot) {
            const int head = u / upr;
            const int i0 = (u - head * upr) << 2;
            float4 a, c;
            load_pair(head * hd + i0, head * hd + half + i0, a, c);
            const float av[4] = {a.x, a.y, a.z, a.w}, cv[4] = {c.x, c.y, c.z, c.w};
            float lo[4], hi[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float cs = cs_table[i0 + j].x, sn = cs_table[i0 + j].y;
                lo[j] = av[j] * cs - cv[j] * sn;
                hi[j] = av[j] * sn + cv[j] * cs;
            }
            if (head < n_heads) {
                T* o = q_out + ((size_t)t * n_heads + head) * hd + i0;
                Pack4<T>::store(o, lo[0], lo[1], lo[2], lo[3]);
                Pack4<T>::store(o + half, hi[0], hi[1], hi[2], hi[3]);
            } else {
                const int hk = head - n_heads;
                if (k_out != nullptr) {
                    T* o = k_out + ((size_t)t * n_kv + hk) * hd + i0;
                    Pack4<T>::store(o, lo[0], lo[1], lo[2], lo[3]);
                    Pack4<T>::store(o + half, hi[0], hi[1], hi[2], hi[3]);
                }
                if (cache_row >= 0) {
                    T* o = k_cache + cache_row + (long long)hk * MF_PAGE * hd + i0;
                    Pack4<T>::store(o, lo[0], lo[1], lo[2], lo[3]);
                    Pack4<T>::store(o + half, hi[0], hi[1], hi[2], hi[3]);
                }
            }
        } else {
            const int idx = u - n_rot;
            const int hk = idx / upv;
            const int e0 = (idx - hk * upv) << 3;
            const int col = (n_heads + n_kv + hk) * hd + e0;
            float4 a, c;
            load_pair(col, col + 4, a, c);
            if (v_out != nullptr) {
                T* o = v_out + ((size_t)t * n_kv + hk) * hd + e0;
                Pack4<T>::store(o, a.x, a.y, a.z, a.w);
                Pack4<T>::store(o + 4, c.x, c.y, c.z, c.w);
            }
            if (cache_row >= 0) {
                T* o = v_cache + cache_row + (long long)hk * MF_PAGE * hd + e0;
                Pack4<T>::store(o, a.x, a.y, a.z, a.w);
                Pack4<T>::store(o + 4, c.x, c.y, c.z, c.w);
            }
        }
    }
}

extern "C" int mf_rope_kvstore(const float* qkv, int n_partials, const float* bias,
                               const int* positions, const int* token_row,
                               const int* seq_end, const double* inv_freq, void* q_out, void* k_out,
                               void* v_out, void* k_cache, void* v_cache, const int* page_table,
                               int table_stride, int ring, int n_tokens, int n_heads, int n_kv,
                               int hd, int rotary_dim, int style, int dtype, unsigned* status,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd % 2 != 0 || rotary_dim % 2 != 0 || rotary_dim > hd || rotary_dim < 0 || rotary_dim > 256)
        return MF_ERR_UNSUPPORTED;
    if (ring % MF_PAGE != 0) return MF_ERR_ARGUMENT;
    const int n_slots = (n_heads + 2 * n_kv) * (hd / 2);
    const int threads = 128;
    // enough blocks to fill the GPU even for a handful of tokens
    int gy = (592 + n_tokens - 1) / n_tokens;
    const int gy_max = (n_slots + threads - 1) / threads;
    if (gy > gy_max) gy = gy_max;
    if (gy < 1) gy = 1;
    const dim3 grid(n_tokens, gy);
    if (inv_freq != nullptr && style == 0 && rotary_dim == hd && hd % 8 == 0 &&
        (dtype == MF_DTYPE_F32 || dtype == MF_DTYPE_BF16)) {
        const int n_units = (n_heads + n_kv) * (hd / 8) + n_kv * (hd / 8);
        int vy = (592 + n_tokens - 1) / n_tokens;
        const int vy_max = (n_units + threads - 1) / threads;
        if (vy > vy_max) vy = vy_max;
        if (vy < 1) vy = 1;
        const dim3 vgrid(n_tokens, vy);
#define MF_ROPE_VEC(T, SPLIT)                                                                    \
    mf_launch(rope_kvstore_vec_kernel<T, SPLIT>, vgrid, dim3(threads), 0, stream, qkv, n_partials, \
              n_tokens, bias, positions, token_row, seq_end, inv_freq, (T*)q_out, (T*)k_out,       \
              (T*)v_out, (T*)k_cache, (T*)v_cache, page_table, table_stride, ring, n_heads, n_kv,  \
              hd, status)
        if (dtype == MF_DTYPE_F32) {
            if (n_partials > 1) MF_ROPE_VEC(float, true); else MF_ROPE_VEC(float, false);
        } else {
            if (n_partials > 1) MF_ROPE_VEC(__nv_bfloat16, true); else MF_ROPE_VEC(__nv_bfloat16, false);
        }
#undef MF_ROPE_VEC
        return MF_LAUNCH_CHECK();
    }
    if (dtype == MF_DTYPE_F32)
        mf_launch(rope_kvstore_kernel<float>, dim3(grid), dim3(threads), 0, stream, 
            qkv, n_partials, n_tokens, bias, positions, token_row, seq_end, inv_freq, (float*)q_out, (float*)k_out,
            (float*)v_out, (float*)k_cache, (float*)v_cache, page_table, table_stride, ring,
            n_heads, n_kv, hd, rotary_dim, style, status);
    else if (dtype == MF_DTYPE_BF16)
        mf_launch(rope_kvstore_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, 
            qkv, n_partials, n_tokens, bias, positions, token_row, seq_end, inv_freq, (__nv_bfloat16*)q_out,
            (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out, (__nv_bfloat16*)k_cache,
            (__nv_bfloat16*)v_cache, page_table, table_stride, ring, n_heads, n_kv, hd,
            rotary_dim, style, status);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// SwiGLU over the fused gate|up projection, silu(z) = z / (1 + exp(-z)), in float32:
//   layout 0 (gate rows then up rows):   out[t][j] = silu(gu[t][j])  * gu[t][nf + j]
//   layout 1 (rows alternate gate, up):  out[t][j] = silu(gu[t][2j]) * gu[t][2j + 1]
// ------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI* __restrict__ gu, TO* __restrict__ out, int nf,
                              long long total, int interleaved) {
    pdl_prologue();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / nf;
        const int j = (int)(idx - t * nf);
        const float g = to_f32(gu[t * 2 * nf + (interleaved ? 2 * j : j)]);
        const float u = to_f32(gu[t * 2 * nf + (interleaved ? 2 * j + 1 : nf + j)]);
        out[idx] = from_f32<TO>(g / (1.0f + expf(-g)) * u);
    }
}

extern "C" int mf_swiglu(const void* gu, int in_dtype, void* out, int out_dtype, int n_rows, int nf,
                         int interleaved, cudaStream_t stream) {
    const long long total = (long long)n_rows * nf;
    if (total <= 0) return 0;
    const int threads = 256;
    const long long cap = (long long)mf_sm_count() * 16;
    const int blocks = (int)((total + threads - 1) / threads < cap ? (total + threads - 1) / threads : cap);
#define MF_SWIGLU(TI, TO) \
    mf_launch(swiglu_kernel<TI, TO>, dim3(blocks), dim3(threads), 0, stream, (const TI*)gu, (TO*)out, nf, total, \
                                                          interleaved)
    if (in_dtype == MF_DTYPE_F32 && out_dtype == MF_DTYPE_F32) MF_SWIGLU(float, float);
    else if (in_dtype == MF_DTYPE_F32 && out_dtype == MF_DTYPE_BF16) MF_SWIGLU(float, __nv_bfloat16);
    else if (in_dtype == MF_DTYPE_BF16 && out_dtype == MF_DTYPE_BF16)
        MF_SWIGLU(__nv_bfloat16, __nv_bfloat16);
    else return MF_ERR_UNSUPPORTED;
#undef MF_SWIGLU
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// row gather of the float32 residual stream: out[r][:] = x[rows[r]][:]
// ------------------------------------------------------------------------------------
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   float* __restrict__ out, int width) {
    pdl_prologue();
    const float* xr = x + (size_t)rows[blockIdx.x] * width;
    float* o = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = xr[i];
}

extern "C" int mf_gather_rows(const float* x, const int* rows, float* out, int n_rows, int width,
                              cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    mf_launch(gather_rows_kernel, dim3(n_rows), dim3(256), 0, stream, x, rows, out, width);
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// cast between float32 and bfloat16 (round to nearest even)
// ------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n) {
    pdl_prologue();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(to_f32(in[i]));
}

extern "C" int mf_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n,
                       cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const long long cap = (long long)mf_sm_count() * 16;
    const int blocks = (int)(want < cap ? want : cap);
    if (in_dtype == MF_DTYPE_F32 && out_dtype == MF_DTYPE_BF16)
        mf_launch(cast_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, 
            (const float*)in, (__nv_bfloat16*)out, n);
    else if (in_dtype == MF_DTYPE_BF16 && out_dtype == MF_DTYPE_F32)
        mf_launch(cast_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(threads), 0, stream, 
            (const __nv_bfloat16*)in, (float*)out, n);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}
