// Attention with grouped query heads, causal by absolute position, optional window.
//
// The formula is the reference's (src/graph/cpu_backend.rs:437-494): head h uses KV head
// h / (n_heads / n_kv); a query at position p sees keys j <= p (and, in a windowed layer,
// p - j < window); s_j = (q . k_j) * scale; softmax over the visible keys; o = sum p_j v_j.
// Scores, the running maximum and sum, and the weighted sum are float32.
//
// This file holds the generic kernel that takes any head size that is a multiple of 16 up
// to 256, float32 or bfloat16, and both sources of keys:
//   * the step's own packed keys/values [token][kv_head][hd] (whole prompts: position j
//     of batch row b lies at token cu_seqlens[b] + j), and
//   * the paged cache (page_table, ring) written by mf_rope_kvstore.
// One warp owns one (query row, head, key chunk): lanes split the keys for the scores and
// split the head dimension for the weighted sum, like the reference's CUDA kernel
// (src/cuda_kernels.cu:673-790) but with the online-softmax state in registers per lane
// pair instead of a full per-lane accumulator, and with key chunks whose boundaries are
// multiples of `chunk` in absolute position, so that a sequence's result does not depend
// on what else is in the batch.  Chunks are merged by mf_attention_combine.
#include "common.cuh"

#define ATT_WARPS 4
#define ATT_MAX_HD 256

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

struct AttnArgs {
    const void* q;            // [rows][n_heads][hd]
    const void* k;            // packed keys  [tokens][n_kv][hd]   (PAGED: cache base)
    const void* v;
    const int* row_seq;       // [rows] batch row of each query
    const int* row_pos;       // [rows] absolute position of each query
    const int* cu_seqlens;    // [B+1] packed source only
    const int* page_table;    // paged source only
    int table_stride;
    int ring;                 // paged source: 0 = linear, else ring length in positions
    void* out;                // [rows][n_heads*hd]            (n_chunks == 1)
    float* partial;           // [rows][n_heads][n_chunks][hd+2] (n_chunks > 1)
    int rows, n_heads, n_kv, hd;
    int window;               // 0 = all earlier keys
    int chunk, n_chunks;
    float scale;
};

template <typename T, bool PAGED>
__global__ void __launch_bounds__(ATT_WARPS * 32) attention_generic_kernel(AttnArgs a) {
    __shared__ float q_s[ATT_WARPS][ATT_MAX_HD];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long item = (long long)blockIdx.x * ATT_WARPS + warp;
    const long long total = (long long)a.rows * a.n_heads * a.n_chunks;
    if (item >= total) return;                        // no block-wide barrier below
    const int chunk_id = (int)(item % a.n_chunks);
    const int head = (int)((item / a.n_chunks) % a.n_heads);
    const int row = (int)(item / ((long long)a.n_chunks * a.n_heads));
    const int hd = a.hd;
    const int hk = head / (a.n_heads / a.n_kv);
    const int b = a.row_seq[row];
    const int pos = a.row_pos[row];
    int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    int hi = pos + 1;
    if (a.n_chunks > 1) {
        lo = max(lo, chunk_id * a.chunk);
        hi = min(hi, (chunk_id + 1) * a.chunk);
    }
    float* part = a.partial
        ? a.partial + (((size_t)row * a.n_heads + head) * a.n_chunks + chunk_id) * (hd + 2)
        : nullptr;
    if (lo >= hi) {                                   // nothing of this chunk is visible
        if (part && lane == 0) { part[0] = -INFINITY; part[1] = 0.0f; }
        return;
    }

    const T* q = (const T*)a.q + ((size_t)row * a.n_heads + head) * hd;
    for (int d = lane; d < hd; d += 32) q_s[warp][d] = to_f32(q[d]) * a.scale;
    __syncwarp();

    const T* kbase = (const T*)a.k;
    const T* vbase = (const T*)a.v;
    const long long packed0 = PAGED ? 0 : (long long)a.cu_seqlens[b];

    float m = -INFINITY, l = 0.0f;
    float acc[ATT_MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < ATT_MAX_HD / 32; ++i) acc[i] = 0.0f;

    for (int j0 = lo; j0 < hi; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j < hi;
        long long off = 0;                            // element offset of key j's row
        if (valid) {
            if (PAGED) {
                const int p_eff = a.ring > 0 ? j % a.ring : j;
                const int page = a.page_table[(size_t)b * a.table_stride + (p_eff >> 6)];
                off = (((long long)page * a.n_kv + hk) * MF_PAGE + (j & (MF_PAGE - 1))) * hd;
            } else {
                off = ((packed0 + j) * a.n_kv + hk) * hd;
            }
        }
        float s = -INFINITY;
        if (valid) {
            const T* kr = kbase + off;
            float dot = 0.0f;
            for (int d = 0; d < hd; d += Vec16<T>::N) {
                float kv[Vec16<T>::N];
                Vec16<T>::load(kr + d, kv);
#pragma unroll
                for (int e = 0; e < Vec16<T>::N; ++e) dot = fmaf(q_s[warp][d + e], kv[e], dot);
            }
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);           // 0 on the first tile (m = -inf)
        const float p = valid ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < ATT_MAX_HD / 32; ++i) acc[i] *= corr;
        const int n_here = min(32, hi - j0);
        for (int jj = 0; jj < n_here; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long voff = __shfl_sync(0xffffffffu, off, jj);
            const T* vr = vbase + voff;
#pragma unroll
            for (int i = 0; i < ATT_MAX_HD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
    }

    if (part) {
        if (lane == 0) { part[0] = m; part[1] = l; }
#pragma unroll
        for (int i = 0; i < ATT_MAX_HD / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) part[2 + d] = acc[i];
        }
    } else {
        T* o = (T*)a.out + ((size_t)row * a.n_heads + head) * hd;
        const float inv = 1.0f / l;
#pragma unroll
        for (int i = 0; i < ATT_MAX_HD / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) o[d] = from_f32<T>(acc[i] * inv);
        }
    }
}

// merges the chunks of one (row, head) in chunk order
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                         int n_chunks, int hd) {
    const size_t rh = blockIdx.x;                     // row * n_heads + head
    const float* p = partial + rh * n_chunks * (hd + 2);
    float m = -INFINITY;
    for (int c = 0; c < n_chunks; ++c) m = fmaxf(m, p[(size_t)c * (hd + 2)]);
    float l = 0.0f;
    for (int c = 0; c < n_chunks; ++c) {
        const float mc = p[(size_t)c * (hd + 2)];
        if (mc > -INFINITY) l += p[(size_t)c * (hd + 2) + 1] * expf(mc - m);
    }
    const float inv = 1.0f / l;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.0f;
        for (int c = 0; c < n_chunks; ++c) {
            const float mc = p[(size_t)c * (hd + 2)];
            if (mc > -INFINITY) o = fmaf(p[(size_t)c * (hd + 2) + 2 + d], expf(mc - m), o);
        }
        out[rh * hd + d] = from_f32<T>(o * inv);
    }
}

static int check_sizes(int n_heads, int n_kv, int hd) {
    if (hd <= 0 || hd % 16 != 0 || hd > ATT_MAX_HD) return MF_ERR_UNSUPPORTED;
    if (n_kv <= 0 || n_heads <= 0 || n_heads % n_kv != 0) return MF_ERR_UNSUPPORTED;
    return 0;
}

// Attention of a step over its own packed keys and values (whole prompts).
extern "C" int mf_attention_packed(const void* q, const void* k, const void* v, const int* row_seq,
                                   const int* row_pos, const int* cu_seqlens, void* out, int rows,
                                   int n_heads, int n_kv, int hd, int window, float scale, int dtype,
                                   cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (int e = check_sizes(n_heads, n_kv, hd)) return e;
    AttnArgs a{};
    a.q = q; a.k = k; a.v = v; a.row_seq = row_seq; a.row_pos = row_pos;
    a.cu_seqlens = cu_seqlens; a.out = out; a.partial = nullptr;
    a.rows = rows; a.n_heads = n_heads; a.n_kv = n_kv; a.hd = hd; a.window = window;
    a.chunk = 0; a.n_chunks = 1; a.scale = scale;
    const long long items = (long long)rows * n_heads;
    const unsigned blocks = (unsigned)((items + ATT_WARPS - 1) / ATT_WARPS);
    if (dtype == MF_DTYPE_F32)
        attention_generic_kernel<float, false><<<blocks, ATT_WARPS * 32, 0, stream>>>(a);
    else if (dtype == MF_DTYPE_BF16)
        attention_generic_kernel<__nv_bfloat16, false><<<blocks, ATT_WARPS * 32, 0, stream>>>(a);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// Attention over the paged cache.  `partial` must hold rows*n_heads*n_chunks*(hd+2) floats
// when n_chunks > 1; chunk c covers absolute positions [c*chunk, (c+1)*chunk).
extern "C" int mf_attention_paged(const void* q, const void* k_cache, const void* v_cache,
                                  const int* row_seq, const int* row_pos, const int* page_table,
                                  int table_stride, int ring, void* out, float* partial, int rows,
                                  int n_heads, int n_kv, int hd, int window, int chunk, int n_chunks,
                                  float scale, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (int e = check_sizes(n_heads, n_kv, hd)) return e;
    if (n_chunks < 1 || (n_chunks > 1 && (partial == nullptr || chunk <= 0))) return MF_ERR_ARGUMENT;
    if (ring % MF_PAGE != 0) return MF_ERR_ARGUMENT;
    AttnArgs a{};
    a.q = q; a.k = k_cache; a.v = v_cache; a.row_seq = row_seq; a.row_pos = row_pos;
    a.page_table = page_table; a.table_stride = table_stride; a.ring = ring;
    a.out = out; a.partial = n_chunks > 1 ? partial : nullptr;
    a.rows = rows; a.n_heads = n_heads; a.n_kv = n_kv; a.hd = hd; a.window = window;
    a.chunk = chunk; a.n_chunks = n_chunks; a.scale = scale;
    const long long items = (long long)rows * n_heads * n_chunks;
    const unsigned blocks = (unsigned)((items + ATT_WARPS - 1) / ATT_WARPS);
    if (dtype == MF_DTYPE_F32)
        attention_generic_kernel<float, true><<<blocks, ATT_WARPS * 32, 0, stream>>>(a);
    else if (dtype == MF_DTYPE_BF16)
        attention_generic_kernel<__nv_bfloat16, true><<<blocks, ATT_WARPS * 32, 0, stream>>>(a);
    else
        return MF_ERR_UNSUPPORTED;
    int e = MF_LAUNCH_CHECK();
    if (e || n_chunks == 1) return e;
    const int threads = hd >= 128 ? 128 : (hd >= 64 ? 64 : 32);
    if (dtype == MF_DTYPE_F32)
        attention_combine_kernel<float><<<rows * n_heads, threads, 0, stream>>>(
            partial, (float*)out, n_chunks, hd);
    else
        attention_combine_kernel<__nv_bfloat16><<<rows * n_heads, threads, 0, stream>>>(
            partial, (__nv_bfloat16*)out, n_chunks, hd);
    return MF_LAUNCH_CHECK();
}
