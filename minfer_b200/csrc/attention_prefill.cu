// Attention of whole prompts on tensor cores (bfloat16, head size 64 or 128): causal,
// grouped query heads, optional window, sequences of unequal lengths packed one after
// another.
//
// Same formula as the generic kernel (src/graph/cpu_backend.rs:437-494 in the reference):
// scores * scale, mask by position, softmax in float32, weighted sum of values.  The
// reference's CUDA kernel gives one warp to a (token, head) and walks the keys one by one
// (src/cuda_kernels.cu:673-790); here a CTA owns 64 queries of one head and walks the keys in
// tiles of 64 with an online softmax: S = Q K^T and O += P V are m16n8k16 bf16 MMAs with
// float32 accumulation, K and V tiles are double-buffered in shared memory by cp.async with
// an XOR swizzle, fragments come out by ldmatrix (transposed for V).  Rows beyond a
// sequence's end are zero-filled, never read from a neighbour.
//
// Positions are the indices inside the sequence: this path serves steps in which every
// sequence starts at position 0.
#include "common.cuh"

#define PF_WARPS 4
#define PF_ROWS 64            // queries per CTA
#define PF_KEYS 64            // keys per tile

struct PrefillArgs {
    const __nv_bfloat16* q;   // [tokens][n_heads][HD]
    const __nv_bfloat16* k;   // [tokens][n_kv][HD]
    const __nv_bfloat16* v;
    const int* cu_seqlens;    // [n_seqs + 1]
    __nv_bfloat16* out;       // [tokens][n_heads * HD]
    int n_heads, n_kv, window;
    float scale_log2;         // scale * log2(e)
};

__device__ __forceinline__ void mma16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                              uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// copies rows [row0, row0+64) of a packed [tokens][heads][HD] tensor (one head) into a
// swizzled [64][HD] tile; rows at or beyond `n_valid` (relative to row0) are zero-filled.
// A thread always copies the same 16-byte column of rows r0, r0 + RPP, ...: its swizzled
// column and its offsets are computed once (TileCopy) and only advanced here.
template <int HD>
struct TileCopy {
    static constexpr int CPR = HD / 8;                    // 16-byte chunks per row
    static constexpr int RPP = PF_WARPS * 32 / CPR;       // rows per pass of the CTA (8 or 16)
    int r0;                                               // first row of this thread
    uint32_t dst_off;                                     // bytes into the tile
    int src_col;                                          // elements into the row
    __device__ __forceinline__ TileCopy(int tid) {
        r0 = tid / CPR;
        const int c = tid % CPR;
        dst_off = (uint32_t)((r0 * CPR + (c ^ (r0 & 7))) * 16);
        src_col = c * 8;
    }
    __device__ __forceinline__ void load(__nv_bfloat16* tile, const __nv_bfloat16* base,
                                         long long row_stride, int n_valid) const {
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(tile) + dst_off;
        const __nv_bfloat16* src = base + (long long)r0 * row_stride + src_col;
#pragma unroll
        for (int j = 0; j < 64 / RPP; ++j) {
            const bool ok = r0 + j * RPP < n_valid;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                         ::"r"(dst + (uint32_t)(j * RPP * CPR * 16)),
                           "l"(ok ? src + (long long)j * RPP * row_stride : base), "r"(ok ? 16 : 0)
                         : "memory");
        }
    }
};

template <int HD>
__global__ void __launch_bounds__(PF_WARPS * 32, 3) attention_prefill_mma_kernel(PrefillArgs a) {
    pdl_prologue();
    constexpr int CPR = HD / 8;
    extern __shared__ __align__(128) uint8_t pf_smem[];
    __nv_bfloat16* k_s = (__nv_bfloat16*)pf_smem;                 // [2][64][HD]
    __nv_bfloat16* v_s = k_s + 2 * 64 * HD;                       // [2][64][HD]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int tok0 = a.cu_seqlens[seq];
    const int len = a.cu_seqlens[seq + 1] - tok0;
    // heavy (late) query tiles first: they have the most keys
    const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int q0 = q_tile * PF_ROWS;
    if (q0 >= len) return;
    const int hk = head / (a.n_heads / a.n_kv);
    const long long q_stride = (long long)a.n_heads * HD, kv_stride = (long long)a.n_kv * HD;
    const __nv_bfloat16* qb = a.q + ((long long)(tok0 + q0) * a.n_heads + head) * HD;
    const __nv_bfloat16* kb = a.k + ((long long)tok0 * a.n_kv + hk) * HD;
    const __nv_bfloat16* vb = a.v + ((long long)tok0 * a.n_kv + hk) * HD;

    const int q_last = min(q0 + PF_ROWS, len) - 1;               // last query position of the tile
    const int kt_begin = a.window > 0 ? max(0, q0 - a.window + 1) / PF_KEYS : 0;
    const int kt_end = q_last / PF_KEYS;                          // inclusive

    const TileCopy<HD> copy(tid);
    copy.load(k_s, kb + (long long)kt_begin * PF_KEYS * kv_stride, kv_stride, len - kt_begin * PF_KEYS);
    copy.load(v_s, vb + (long long)kt_begin * PF_KEYS * kv_stride, kv_stride, len - kt_begin * PF_KEYS);
    asm volatile("cp.async.commit_group;" ::: "memory");

    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    const int row_g = q0 + warp * 16 + g;                         // this thread's rows: row_g, row_g + 8
    // query fragments straight from global memory (once per CTA; rows beyond the end are zero)
    uint32_t qa[HD / 16][4];
    {
        const __nv_bfloat16* q_lo = qb + (long long)(warp * 16 + g) * q_stride + 2 * t;
        const __nv_bfloat16* q_hi = q_lo + 8 * q_stride;
        const bool lo_ok = row_g < len, hi_ok = row_g + 8 < len;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            qa[ks][0] = lo_ok ? *reinterpret_cast<const uint32_t*>(q_lo + 16 * ks) : 0u;
            qa[ks][1] = hi_ok ? *reinterpret_cast<const uint32_t*>(q_hi + 16 * ks) : 0u;
            qa[ks][2] = lo_ok ? *reinterpret_cast<const uint32_t*>(q_lo + 16 * ks + 8) : 0u;
            qa[ks][3] = hi_ok ? *reinterpret_cast<const uint32_t*>(q_hi + 16 * ks + 8) : 0u;
        }
    }

    // ldmatrix addresses: a lane's row offset and its swizzled 16-byte column per k-step (keys)
    // or per pair of output columns (values), computed once
    const uint32_t k_lane = (uint32_t)((((lane >> 4) * 8 + (lane & 7)) * CPR) * 16);
    const uint32_t v_lane = (uint32_t)(((((lane >> 3) & 1) * 8 + (lane & 7)) * CPR) * 16);
    uint32_t k_col[HD / 16], v_col[HD / 16];
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) {
        k_col[i] = (uint32_t)(((2 * i + ((lane >> 3) & 1)) ^ (lane & 7)) * 16);
        v_col[i] = (uint32_t)(((2 * i + (lane >> 4)) ^ (lane & 7)) * 16);
    }
    const uint32_t k_s_addr = (uint32_t)__cvta_generic_to_shared(k_s);
    const uint32_t v_s_addr = (uint32_t)__cvta_generic_to_shared(v_s);

    for (int kt = kt_begin; kt <= kt_end; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        if (kt < kt_end) {                                        // prefetch the next tile
            const int nb = buf ^ 1;
            const long long off = (long long)(kt + 1) * PF_KEYS * kv_stride;
            copy.load(k_s + nb * 64 * HD, kb + off, kv_stride, len - (kt + 1) * PF_KEYS);
            copy.load(v_s + nb * 64 * HD, vb + off, kv_stride, len - (kt + 1) * PF_KEYS);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();

        // S[16][64] = Q K^T
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
        const uint32_t ks_base = k_s_addr + (uint32_t)(buf * 64 * HD * 2) + k_lane;
        // k-step outermost: consecutive MMAs go to different accumulators, so none waits for
        // the one before it
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {                      // pairs of 8-key tiles
                uint32_t b0, b1, b2, b3;
                ldsm_x4(ks_base + k_col[ks] + (uint32_t)(np * 16 * CPR * 16), b0, b1, b2, b3);
                mma16816(s[2 * np], qa[ks], b0, b1);
                mma16816(s[2 * np + 1], qa[ks], b2, b3);
            }
        }

        // mask by position where the tile touches the diagonal, the window's edge or the end
        const int key0 = kt * PF_KEYS;
        const bool need_mask = key0 + PF_KEYS - 1 > q0 + warp * 16 ||
                               (a.window > 0 && key0 < q0 + warp * 16 + 15 - a.window + 1) ||
                               key0 + PF_KEYS > len;
        if (need_mask) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + nt * 8 + 2 * t + (e & 1);
                    const int row = row_g + (e >> 1) * 8;
                    const bool vis = key <= row && key < len &&
                                     (a.window == 0 || row - key < a.window);
                    if (!vis) s[nt][e] = -INFINITY;
                }
            }
        }
        // online softmax (base 2)
        float m_new[2] = {m_r[0], m_r[1]};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            m_new[0] = fmaxf(m_new[0], fmaxf(s[nt][0], s[nt][1]));
            m_new[1] = fmaxf(m_new[1], fmaxf(s[nt][2], s[nt][3]));
        }
        float corr[2], m_scaled[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
            // a row with nothing visible yet keeps m = -inf; use 0 as its offset so that
            // exp2(-inf - 0) = 0 and no inf - inf appears
            m_scaled[r] = m_new[r] == -INFINITY ? 0.0f : m_new[r] * a.scale_log2;
            corr[r] = m_r[r] == -INFINITY ? 0.0f : exp2f(m_r[r] * a.scale_log2 - m_scaled[r]);
            m_r[r] = m_new[r];
            l_r[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        uint32_t pa[4][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = exp2f(s[nt][e] * a.scale_log2 - m_scaled[e >> 1]);
                l_r[e >> 1] += p[e];
            }
            pa[nt >> 1][(nt & 1) * 2 + 0] = pack2(p[0], p[1]);
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack2(p[2], p[3]);
        }
        // O += P V
        const uint32_t vs_base = v_s_addr + (uint32_t)(buf * 64 * HD * 2) + v_lane;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int np = 0; np < HD / 16; ++np) {
                uint32_t r0, r1, r2, r3;
                ldsm_x4_trans(vs_base + v_col[np] + (uint32_t)(ks * 16 * CPR * 16), r0, r1, r2, r3);
                mma16816(o[2 * np], pa[ks], r0, r1);
                mma16816(o[2 * np + 1], pa[ks], r2, r3);
            }
        }
        __syncthreads();                                          // the buffer may be refilled now
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 1);
        l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 2);
    }
    const float inv0 = 1.0f / l_r[0], inv1 = 1.0f / l_r[1];
    const int r0 = row_g, r1 = row_g + 8;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        const int d = nt * 8 + 2 * t;
        if (r0 < len)
            *reinterpret_cast<uint32_t*>(a.out + ((long long)(tok0 + r0) * a.n_heads + head) * HD + d) =
                pack2(o[nt][0] * inv0, o[nt][1] * inv0);
        if (r1 < len)
            *reinterpret_cast<uint32_t*>(a.out + ((long long)(tok0 + r1) * a.n_heads + head) * HD + d) =
                pack2(o[nt][2] * inv1, o[nt][3] * inv1);
    }
}

template <int HD>
static int launch_prefill(const PrefillArgs& a, int n_seqs, int max_len, cudaStream_t stream) {
    constexpr int smem = 4 * 64 * HD * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_mma_kernel<HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((max_len + PF_ROWS - 1) / PF_ROWS, a.n_heads, n_seqs);
    mf_launch(attention_prefill_mma_kernel<HD>, dim3(grid), dim3(PF_WARPS * 32), smem, stream, a);
    return MF_LAUNCH_CHECK();
}

// q [tokens][n_heads][hd], k/v [tokens][n_kv][hd], out [tokens][n_heads*hd], all bfloat16;
// sequence b holds tokens cu_seqlens[b] .. cu_seqlens[b+1]-1 at positions 0, 1, 2, ...
extern "C" int mf_attention_prefill_mma(const void* q, const void* k, const void* v,
                                        const int* cu_seqlens, void* out, int n_seqs, int max_len,
                                        int n_heads, int n_kv, int hd, int window, float scale,
                                        cudaStream_t stream) {
    if (n_seqs <= 0 || max_len <= 0) return 0;
    if ((hd != 64 && hd != 128) || n_kv <= 0 || n_heads % n_kv != 0) return MF_ERR_UNSUPPORTED;
    if (n_heads > 65535 || n_seqs > 65535) return MF_ERR_UNSUPPORTED;
    PrefillArgs a;
    a.q = (const __nv_bfloat16*)q; a.k = (const __nv_bfloat16*)k; a.v = (const __nv_bfloat16*)v;
    a.cu_seqlens = cu_seqlens; a.out = (__nv_bfloat16*)out;
    a.n_heads = n_heads; a.n_kv = n_kv; a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    return hd == 64 ? launch_prefill<64>(a, n_seqs, max_len, stream)
                    : launch_prefill<128>(a, n_seqs, max_len, stream);
}
