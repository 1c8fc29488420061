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
#include <cuda.h>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

#define MF_ERR_NO_TENSORMAP 2003
#define MF_ERR_TENSORMAP 2004

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
    unsigned* status;         // device status word (the kernel with bounded waits only)
    int old_keys_final;       // 1: of the keys a row sees, only the one at its own position is
                              // written by a kernel of this step (one new token per sequence)
};

template <typename T, bool PAGED>
__global__ void __launch_bounds__(ATT_WARPS * 32) attention_generic_kernel(AttnArgs a) {
    pdl_prologue();
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

// merges the chunks of one (row, head) in chunk order.  The chunks' maxima and sums are
// fetched once (a load per thread), the factors exp(m_c - m) computed once per chunk; then
// every thread sums its output dimension over the chunks with loads that do not wait for one
// another.  Dynamic shared memory: 2 * n_chunks floats.
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                         int n_chunks, int hd) {
    pdl_prologue();
    extern __shared__ float comb_s[];
    float* f_s = comb_s;                              // m_c, then the factor of chunk c
    float* l_s = comb_s + n_chunks;
    __shared__ float red_s[33];
    const size_t rh = blockIdx.x;                     // row * n_heads + head
    const size_t stride = (size_t)(hd + 2);
    const float* p = partial + rh * n_chunks * stride;
    if (n_chunks <= 16) {
        // few chunks: every thread reads the maxima and sums itself (no barrier at all) and
        // asks for its first output dimension's values in the same breath: one round trip
        float mc[16], lc[16], oc[16];
        const int d0 = threadIdx.x;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            if (c < n_chunks) {
                mc[c] = p[(size_t)c * stride];
                lc[c] = p[(size_t)c * stride + 1];
                oc[c] = d0 < hd ? p[(size_t)c * stride + 2 + d0] : 0.0f;
            }
        }
        float m = -INFINITY;
#pragma unroll
        for (int c = 0; c < 16; ++c)
            if (c < n_chunks) m = fmaxf(m, mc[c]);
        float l = 0.0f;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            if (c < n_chunks) {
                mc[c] = mc[c] > -INFINITY ? expf(mc[c] - m) : 0.0f;     // the chunk's factor
                if (mc[c] > 0.0f) l += lc[c] * mc[c];
            }
        }
        const float inv = 1.0f / l;
        for (int d = d0; d < hd; d += blockDim.x) {
            float o = 0.0f;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                if (c < n_chunks) {
                    const float v = d == d0 ? oc[c] : p[(size_t)c * stride + 2 + d];
                    if (mc[c] > 0.0f) o = fmaf(v, mc[c], o);
                }
            }
            out[rh * hd + d] = from_f32<T>(o * inv);
        }
        return;
    }
    float m_l = -INFINITY;
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
        const float mc = p[(size_t)c * stride];
        f_s[c] = mc;
        l_s[c] = p[(size_t)c * stride + 1];
        m_l = fmaxf(m_l, mc);
    }
    const float m = block_max(m_l, red_s);            // (also orders the writes above)
    float l_l = 0.0f;
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
        const float mc = f_s[c];
        const float f = mc > -INFINITY ? expf(mc - m) : 0.0f;
        f_s[c] = f;
        l_l += l_s[c] * f;
    }
    const float l = block_sum(l_l, red_s);
    const float inv = 1.0f / l;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll 8
        for (int c = 0; c < n_chunks; ++c) {
            const float f = f_s[c];
            if (f > 0.0f) o = fmaf(p[(size_t)c * stride + 2 + d], f, o);
        }
        out[rh * hd + d] = from_f32<T>(o * inv);
    }
}

// ------------------------------------------------------------------------------------------
// Decoding over the paged cache on tensor cores (bfloat16, head size 64 or 128, up to 16
// query heads per key/value head).
//
// One CTA owns (key chunk, key/value head, query row).  A chunk is a multiple of 256 positions
// and is walked in blocks of 256; each of the eight warps takes 32 keys of a block and carries
// its running maximum, sum and output from block to block.  The caller sizes the chunks (one
// block when there are many rows, several when the context is long and the rows are few).
// The group's query heads are the 16 rows of an m16n8k16 MMA, so
// a key or value element is read once for the whole group (the reference's kernel re-reads
// the cache for every query head: src/cuda_kernels.cu:673-790).  Keys go from global memory
// straight into MMA fragments (16-byte loads; k is permuted the same way in both operands,
// which a dot product does not see); values are staged in shared memory by cp.async with an
// XOR swizzle and read transposed by ldmatrix.  Scores, maxima and sums are float32; the
// probabilities are rounded to bfloat16 for the second product.  The warps' results are
// merged in shared memory in warp order and written as one partial per chunk, which
// attention_combine_kernel merges in chunk order; a row with a single chunk is written out
// directly.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16_16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

#define DEC_WARPS 8           // warps per CTA; each takes DEC_KEYS keys of the 256-key chunk
#define DEC_KEYS 32

// MINB: CTAs per SM the registers are cut for.  Two (128 registers) are faster while all CTAs
// fit on the GPU at once; with many rounds of CTAs a third one per SM (80 registers) keeps
// more loads in flight (batch 64: 2.8 % of a step).
// LOOP: the chunk may hold more than one block of 256 keys.
template <int HD, int MINB, bool LOOP>
__global__ void __launch_bounds__(DEC_WARPS * 32, MINB) attention_decode_mma_kernel(AttnArgs a) {
    pdl_prologue();
    constexpr int CPR = HD / 8;                       // 16-byte chunks per row
    extern __shared__ __align__(128) uint8_t dec_smem[];
    // values [DEC_WARPS][DEC_KEYS][HD] bf16, swizzled; once every warp is done with its values
    // the same memory holds the warps' results [DEC_WARPS][16][HD] float32
    // (rows padded by 8 floats: a warp's float2 stores of 8 rows then spread over all banks)
    constexpr int OS = HD + 8;
    __nv_bfloat16* v_s = (__nv_bfloat16*)dec_smem;
    float* o_s = (float*)dec_smem;
    float* ml_s = (float*)(dec_smem + DEC_WARPS * 16 * OS * 4);          // [DEC_WARPS][16][2]
    float* f_s = ml_s + DEC_WARPS * 16 * 2;                              // [DEC_WARPS][16] merge factors
    float* l_s = f_s + DEC_WARPS * 16;                                   // [16] the chunk's sums

    const int chunk_id = blockIdx.x, hk = blockIdx.y, row = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int G = a.n_heads / a.n_kv;
    const int b = a.row_seq[row];
    const int pos = a.row_pos[row];
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int hi = pos + 1;
    // the CTA's chunk: a.chunk keys (a multiple of 256), walked in blocks of 256; every warp
    // carries its running maximum, sum and output from block to block
    const int chunk_lo = chunk_id * a.chunk;
    const size_t part_stride = (size_t)(HD + 2);
    float* part0 = a.partial + (((size_t)row * a.n_heads + (size_t)hk * G) * a.n_chunks + chunk_id) * part_stride;
    if (max(lo, chunk_lo) >= min(hi, chunk_lo + a.chunk)) {       // nothing of this chunk is visible
        if (tid < G) {
            float* p = part0 + (size_t)tid * a.n_chunks * part_stride;
            p[0] = -INFINITY;
            p[1] = 0.0f;
        }
        return;
    }

    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }

    for (int c_lo = chunk_lo; c_lo == chunk_lo || (LOOP && c_lo < chunk_lo + a.chunk && c_lo < hi); c_lo += 256) {
    const int j0 = c_lo + warp * DEC_KEYS;            // first position of this warp's keys
    const int w_lo = max(lo, j0), w_hi = min(hi, j0 + DEC_KEYS);
    const bool active = w_lo < w_hi;
    if (active) {
        __syncwarp();                                 // the block before is done with the warp's values
        const int p_eff = a.ring > 0 ? j0 % a.ring : j0;
        const int page = a.page_table[(size_t)b * a.table_stride + (p_eff >> 6)];
        const size_t tile = (((size_t)page * a.n_kv + hk) * MF_PAGE + (j0 & (MF_PAGE - 1))) * HD;
        const __nv_bfloat16* kp = (const __nv_bfloat16*)a.k + tile;
        const __nv_bfloat16* vp = (const __nv_bfloat16*)a.v + tile;
        __nv_bfloat16* vw = v_s + (size_t)warp * DEC_KEYS * HD;
        // values -> shared memory (asynchronously; the scores are computed meanwhile)
        {
            const uint32_t vw_addr = (uint32_t)__cvta_generic_to_shared(vw);
#pragma unroll
            for (int it = 0; it < DEC_KEYS * CPR / 32; ++it) {
                const int i = it * 32 + lane;
                const int r = i / CPR, c = i % CPR;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                             ::"r"(vw_addr + (uint32_t)((r * CPR + (c ^ (r & 7))) * 16)),
                               "l"(vp + (size_t)i * 8) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }

        // query fragments: rows g and g+8 of the group (zero beyond the group's heads)
        uint32_t qa[HD / 16][4];
        const __nv_bfloat16* qrow = (const __nv_bfloat16*)a.q + ((size_t)row * a.n_heads + (size_t)hk * G) * HD;
#pragma unroll
        for (int s = 0; s < HD / 32; ++s) {
            uint4 q0 = make_uint4(0, 0, 0, 0), q1 = make_uint4(0, 0, 0, 0);
            if (g < G) q0 = *reinterpret_cast<const uint4*>(qrow + (size_t)g * HD + 32 * s + 8 * t);
            if (g + 8 < G) q1 = *reinterpret_cast<const uint4*>(qrow + (size_t)(g + 8) * HD + 32 * s + 8 * t);
            qa[2 * s][0] = q0.x; qa[2 * s][1] = q1.x; qa[2 * s][2] = q0.y; qa[2 * s][3] = q1.y;
            qa[2 * s + 1][0] = q0.z; qa[2 * s + 1][1] = q1.z; qa[2 * s + 1][2] = q0.w; qa[2 * s + 1][3] = q1.w;
        }

        // scores S[16 heads][32 keys]: all key loads first (16 independent 16-byte loads a thread)
        constexpr int NT = DEC_KEYS / 8;
        float sacc[NT][4];
        uint4 kv[NT][HD / 32];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const __nv_bfloat16* kr = kp + (size_t)(nt * 8 + g) * HD + 8 * t;
#pragma unroll
            for (int s = 0; s < HD / 32; ++s) kv[nt][s] = __ldg(reinterpret_cast<const uint4*>(kr + 32 * s));
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.0f;
        // k-step outermost: consecutive MMAs go to different accumulators
#pragma unroll
        for (int s = 0; s < HD / 32; ++s) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(sacc[nt], qa[2 * s], kv[nt][s].x, kv[nt][s].y);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(sacc[nt], qa[2 * s + 1], kv[nt][s].z, kv[nt][s].w);
        }
        // scale (to base 2), mask by position, row maxima (on top of the blocks before)
        const float sl2 = a.scale * 1.4426950408889634f;
        const float m_old[2] = {m_r[0], m_r[1]};
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = j0 + nt * 8 + 2 * t + (e & 1);
                const float sv = (key >= w_lo && key < w_hi) ? sacc[nt][e] * sl2 : -INFINITY;
                sacc[nt][e] = sv;
                m_r[e >> 1] = fmaxf(m_r[e >> 1], sv);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            m_r[r] = fmaxf(m_r[r], __shfl_xor_sync(0xffffffffu, m_r[r], 1));
            m_r[r] = fmaxf(m_r[r], __shfl_xor_sync(0xffffffffu, m_r[r], 2));
        }
        if (LOOP && c_lo != chunk_lo) {
            // what the warp holds from earlier blocks comes down to the new maxima
            const float c0 = m_old[0] > -INFINITY ? exp2f(m_old[0] - m_r[0]) : 0.0f;
            const float c1 = m_old[1] > -INFINITY ? exp2f(m_old[1] - m_r[1]) : 0.0f;
            l_r[0] *= c0; l_r[1] *= c1;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
        }
        uint32_t pa[NT / 2][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = exp2f(sacc[nt][e] - m_r[e >> 1]);
                l_r[e >> 1] += p[e];
            }
            pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
        // O[16 heads][HD] = P[16][32] V[32][HD]
        const uint32_t vbase = (uint32_t)__cvta_generic_to_shared(vw);
#pragma unroll
        for (int ks = 0; ks < DEC_KEYS / 16; ++ks) {
            const int key = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
            for (int np = 0; np < HD / 16; ++np) {
                const int dchunk = 2 * np + (lane >> 4);
                const uint32_t addr = vbase + (uint32_t)((key * CPR + (dchunk ^ (key & 7))) * 16);
                uint32_t r0, r1, r2, r3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
                mma_bf16_16816(o[2 * np], pa[ks], r0, r1);
                mma_bf16_16816(o[2 * np + 1], pa[ks], r2, r3);
            }
        }
    }
    }   // blocks of the chunk
    // the four lanes of a row each hold a part of its sum
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 1);
        l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 2);
    }
    // maxima (base-2 units) and sums of every warp, then the factors that bring them to the
    // chunk's maximum
    if (t == 0) {
        ml_s[(warp * 16 + g) * 2 + 0] = m_r[0]; ml_s[(warp * 16 + g) * 2 + 1] = l_r[0];
        ml_s[(warp * 16 + g + 8) * 2 + 0] = m_r[1]; ml_s[(warp * 16 + g + 8) * 2 + 1] = l_r[1];
    }
    __syncthreads();                                  // also: every warp is done reading its values
    if (tid < 16) {
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, ml_s[(w * 16 + tid) * 2]);
        float l = 0.0f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float mw = ml_s[(w * 16 + tid) * 2];
            const float f = mw > -INFINITY ? exp2f(mw - m) : 0.0f;
            f_s[w * 16 + tid] = f;
            l += ml_s[(w * 16 + tid) * 2 + 1] * f;
        }
        l_s[tid] = l;
        if (tid < G && a.n_chunks > 1) {
            float* p = part0 + (size_t)tid * a.n_chunks * part_stride;
            p[0] = m * 0.6931471805599453f;           // back to natural-log units for the merge
            p[1] = l;
        }
    }
    float* ow = o_s + (size_t)warp * 16 * OS;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        *reinterpret_cast<float2*>(ow + (size_t)g * OS + nt * 8 + 2 * t) = make_float2(o[nt][0], o[nt][1]);
        if (G > 8)      // rows 8-15 hold heads only in groups of more than eight
            *reinterpret_cast<float2*>(ow + (size_t)(g + 8) * OS + nt * 8 + 2 * t) = make_float2(o[nt][2], o[nt][3]);
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += DEC_WARPS * 32) {
        const int r = idx / HD, d = idx - r * HD;
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) acc = fmaf(o_s[((size_t)w * 16 + r) * OS + d], f_s[w * 16 + r], acc);
        if (a.n_chunks > 1)
            part0[(size_t)r * a.n_chunks * part_stride + 2 + d] = acc;
        else        // the only chunk: the result itself, no merge kernel follows
            ((__nv_bfloat16*)a.out)[((size_t)row * a.n_heads + (size_t)hk * G + r) * HD + d] =
                __float2bfloat16(acc / l_s[r]);
    }
}

#define MF_MAX_DEVICES 64

// The kernel's dynamic shared memory is opened once per device (a function attribute belongs
// to the device that is current when it is set).
template <int HD, int MINB, bool LOOP>
static int configure_decode_mma() {
    constexpr int smem = DEC_WARPS * 16 * (HD + 8) * 4 + DEC_WARPS * 16 * 3 * 4 + 16 * 4;
    static bool configured[MF_MAX_DEVICES] = {false};
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= MF_MAX_DEVICES) return MF_ERR_UNSUPPORTED;
    if (!configured[device]) {
        e = cudaFuncSetAttribute(attention_decode_mma_kernel<HD, MINB, LOOP>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured[device] = true;
    }
    return 0;
}

// every variant mf_attention_paged may pick without a status word, for the current device
static int configure_decode_mma_all() {
    if (int e = configure_decode_mma<64, 2, false>()) return e;
    if (int e = configure_decode_mma<64, 3, false>()) return e;
    if (int e = configure_decode_mma<64, 2, true>()) return e;
    if (int e = configure_decode_mma<128, 2, false>()) return e;
    if (int e = configure_decode_mma<128, 3, false>()) return e;
    return configure_decode_mma<128, 2, true>();
}

template <int HD, int MINB, bool LOOP>
static int launch_decode_mma_as(const AttnArgs& a, cudaStream_t stream) {
    constexpr int smem = DEC_WARPS * 16 * (HD + 8) * 4 + DEC_WARPS * 16 * 3 * 4 + 16 * 4;
    static_assert(DEC_WARPS * DEC_KEYS * HD * 2 <= DEC_WARPS * 16 * (HD + 8) * 4, "values fit the staging area");
    static_assert(DEC_WARPS * DEC_KEYS == 256, "a CTA walks its chunk in blocks of 256 keys");
    if (int e = configure_decode_mma<HD, MINB, LOOP>()) return e;
    dim3 grid(a.n_chunks, a.n_kv, a.rows);
    mf_launch(attention_decode_mma_kernel<HD, MINB, LOOP>, dim3(grid), dim3(DEC_WARPS * 32), smem, stream, a);
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// The same decoding attention for chunks of several pages: the keys and values of a chunk come
// through a ring in shared memory that a producer warp keeps filled by TMA, a page (64
// positions of one key/value head: one stage) at a time, so that the next pages are in flight
// while the four consumer warps work on this one.  (In the kernel above a warp asks for its
// next keys only when it is done with these: with long chunks the loads in flight do not cover
// the memory latency.)
//
//   warp 4       producer: looks up the chunk's pages (32 table entries a time, one per lane),
//                waits for a stage to be free and issues the copies of its K and V tiles
//                (tensor maps over the layer's cache [pages * kv_heads * 64][HD], boxes of
//                64 x 64 elements with the 128-byte swizzle)
//   warps 0-3    consumers: warp w owns keys 16w..16w+15 of every page.  Scores on mma.sync
//                with the keys read by ldmatrix, running maximum and sum in float32,
//                probabilities rounded to bfloat16, values read transposed by ldmatrix.  A warp
//                frees a stage with one arrival; it never waits for the other warps.
// At the chunk's end the four warps' results are merged in warp order in shared memory (over
// the ring, which is idle by then) exactly like the eight warps above.  Waits are bounded.
// ------------------------------------------------------------------------------------------
#define RING_CONSUMERS 4
#define RING_THREADS ((RING_CONSUMERS + 1) * 32)
#define RING_MAX_SPIN (1u << 24)
#define RING_MAX_WAIT_NS 2000000000ull

__device__ __forceinline__ uint32_t ring_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool ring_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// false: the wait ran out (or another thread's did); the flag tells everyone to stop
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it < RING_MAX_SPIN; ++it) {
        if (ring_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if ((it & 1023u) == 1023u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > RING_MAX_WAIT_NS) break;
        }
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void ring_tma(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

template <int HD, int STAGES, int MINB>
__global__ void __launch_bounds__(RING_THREADS, MINB)
attention_decode_ring_kernel(const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, AttnArgs a) {
    // Positions and page tables are copied in before the step's first kernel starts, and (with
    // old_keys_final) the pages below a row's own position were written by earlier steps: the
    // producer asks for those before it waits for the kernel before this one, which wrote the
    // newest key and the queries.  Everything else comes after the wait.
    pdl_launch_dependents();
    constexpr int HALF_BYTES = MF_PAGE * 128;          // one box: 64 keys x 64 elements
    constexpr int KV_BYTES = (HD / 64) * HALF_BYTES;   // the keys (or the values) of a page
    constexpr int STAGE_BYTES = 2 * KV_BYTES;
    constexpr int OS = HD + 8;
    extern __shared__ uint8_t ring_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)ring_raw + 1023) & ~(uintptr_t)1023);
    float* o_s = (float*)smem;                                           // over the ring, at the end
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);           // full[S], empty[S]
    float* ml_s = (float*)(bars + 2 * STAGES);                           // [consumers][16][2]
    float* f_s = ml_s + RING_CONSUMERS * 16 * 2;                         // [consumers][16]
    float* l_s = f_s + RING_CONSUMERS * 16;                              // [16]
    volatile int* abort_flag = (volatile int*)(l_s + 16);

    const int chunk_id = blockIdx.x, hk = blockIdx.y, row = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int G = a.n_heads / a.n_kv;
    const int b = a.row_seq[row];
    const int pos = a.row_pos[row];
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int hi = pos + 1;
    const int chunk_lo = chunk_id * a.chunk;
    const int k_lo = max(lo, chunk_lo), k_hi = min(hi, chunk_lo + a.chunk);
    const size_t part_stride = (size_t)(HD + 2);
    float* part0 = a.partial + (((size_t)row * a.n_heads + (size_t)hk * G) * a.n_chunks + chunk_id) * part_stride;
    if (k_lo >= k_hi) {                               // nothing of this chunk is visible
        pdl_wait();
        if (tid < G) {
            float* p = part0 + (size_t)tid * a.n_chunks * part_stride;
            p[0] = -INFINITY;
            p[1] = 0.0f;
        }
        return;
    }
    const int first = k_lo & ~(MF_PAGE - 1);          // position of the first page to visit
    const int n_tiles = (k_hi - first + MF_PAGE - 1) / MF_PAGE;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ring_smem(&bars[s])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;"
                         ::"r"(ring_smem(&bars[STAGES + s])), "r"(RING_CONSUMERS));
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == RING_CONSUMERS) {
        // ---- producer ---------------------------------------------------------------------
        bool ok = true, waited = false;
        const bool early = a.old_keys_final != 0 && a.ring == 0;
        for (int base = 0; base < n_tiles; base += 32) {
            int page = 0;
            if (base + lane < n_tiles) {
                const int p = first + (base + lane) * MF_PAGE;
                const int p_eff = a.ring > 0 ? p % a.ring : p;
                page = a.page_table[(size_t)b * a.table_stride + (p_eff >> 6)];
            }
            const int cnt = min(32, n_tiles - base);
            // the next few old pages beyond the ring: asked for in L2 now, so that their turn in
            // the ring is not a trip to HBM
            if (base == 0 && early && lane >= STAGES && lane < 2 * STAGES && lane < n_tiles &&
                first + (lane + 1) * MF_PAGE <= pos) {
                const int y = (page * a.n_kv + hk) * MF_PAGE;
#pragma unroll
                for (int h = 0; h < HD / 64; ++h) {
                    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                                 ::"l"(&map_k), "r"(h * 64), "r"(y) : "memory");
                    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                                 ::"l"(&map_v), "r"(h * 64), "r"(y) : "memory");
                }
            }
            for (int i = 0; i < cnt; ++i) {
                const int pg = __shfl_sync(0xffffffffu, page, i);
                if (lane == 0 && ok) {
                    const int n = base + i, s = n % STAGES;
                    const uint32_t ph = (uint32_t)(n / STAGES) & 1u;
                    // a page that ends below the row's position holds no key of this step
                    if (!waited && !(early && first + (n + 1) * MF_PAGE <= pos)) {
                        pdl_wait();
                        waited = true;
                    }
                    ok = ring_wait(ring_smem(&bars[STAGES + s]), ph ^ 1u, abort_flag);
                    if (ok) {
                        const uint32_t full = ring_smem(&bars[s]);
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                                     ::"r"(full), "r"((uint32_t)STAGE_BYTES) : "memory");
                        const uint32_t dst = ring_smem(smem + (size_t)s * STAGE_BYTES);
                        const int y = (pg * a.n_kv + hk) * MF_PAGE;
#pragma unroll
                        for (int h = 0; h < HD / 64; ++h) {
                            ring_tma(dst + h * HALF_BYTES, &map_k, h * 64, y, full);
                            ring_tma(dst + KV_BYTES + h * HALF_BYTES, &map_v, h * 64, y, full);
                        }
                    }
                }
            }
        }
        if (lane == 0 && !waited) pdl_wait();
        if (lane == 0 && !ok && a.status) atomicOr(a.status, MF_STATUS_WAIT_TIMEOUT);
        return;
    }
    pdl_wait();

    // ---- consumers ----------------------------------------------------------------------------
    // query fragments: rows g and g+8 of the group (zero beyond the group's heads)
    uint32_t qa[HD / 16][4];
    {
        const __nv_bfloat16* qrow = (const __nv_bfloat16*)a.q + ((size_t)row * a.n_heads + (size_t)hk * G) * HD;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            const __nv_bfloat16* q0 = qrow + (size_t)g * HD + 16 * kk + 2 * t;
            const __nv_bfloat16* q1 = qrow + (size_t)(g + 8) * HD + 16 * kk + 2 * t;
            qa[kk][0] = g < G ? *reinterpret_cast<const uint32_t*>(q0) : 0u;
            qa[kk][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(q1) : 0u;
            qa[kk][2] = g < G ? *reinterpret_cast<const uint32_t*>(q0 + 8) : 0u;
            qa[kk][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(q1 + 8) : 0u;
        }
    }
    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    const float sl2 = a.scale * 1.4426950408889634f;
    const uint32_t ring_base = ring_smem(smem);
    bool ok = true;

    for (int n = 0; n < n_tiles; ++n) {
        const int s = n % STAGES;
        const uint32_t ph = (uint32_t)(n / STAGES) & 1u;
        ok = __all_sync(0xffffffffu, ring_wait(ring_smem(&bars[s]), ph, abort_flag));
        if (!ok) break;
        const int j0 = first + n * MF_PAGE + warp * 16;            // first position of this warp's keys
        const int w_lo = max(k_lo, j0), w_hi = min(k_hi, j0 + 16);
        if (w_lo < w_hi) {
            const uint32_t kaddr = ring_base + (uint32_t)(s * STAGE_BYTES);
            const uint32_t vaddr = kaddr + KV_BYTES;
            // scores S[16 heads][16 keys]
            // (two accumulators per key tile, for even and odd steps along the head: half as
            // long a chain of dependent MMAs; added below)
            float sacc[2][4], sodd[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.0f;
                sodd[nt][0] = sodd[nt][1] = sodd[nt][2] = sodd[nt][3] = 0.0f;
            }
#pragma unroll
            for (int ks2 = 0; ks2 < HD / 32; ++ks2) {
                const int c = 4 * ks2 + (lane >> 3);              // 16-byte piece of a key's row
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const int r = warp * 16 + nt * 8 + (lane & 7);
                    const uint32_t addr = kaddr + (uint32_t)((c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4));
                    uint32_t r0, r1, r2, r3;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
                    mma_bf16_16816(sacc[nt], qa[2 * ks2], r0, r1);
                    mma_bf16_16816(sodd[nt], qa[2 * ks2 + 1], r2, r3);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sacc[nt][e] += sodd[nt][e];
            }
            // scale (to base 2), mask by position, row maxima on top of the pages before
            const float m_old[2] = {m_r[0], m_r[1]};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = j0 + nt * 8 + 2 * t + (e & 1);
                    const float sv = (key >= w_lo && key < w_hi) ? sacc[nt][e] * sl2 : -INFINITY;
                    sacc[nt][e] = sv;
                    m_r[e >> 1] = fmaxf(m_r[e >> 1], sv);
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                m_r[r] = fmaxf(m_r[r], __shfl_xor_sync(0xffffffffu, m_r[r], 1));
                m_r[r] = fmaxf(m_r[r], __shfl_xor_sync(0xffffffffu, m_r[r], 2));
            }
            if (__any_sync(0xffffffffu, m_r[0] != m_old[0] || m_r[1] != m_old[1])) {
                // what the warp holds from earlier pages comes down to the new maxima
                const float c0 = m_old[0] > -INFINITY ? exp2f(m_old[0] - m_r[0]) : 0.0f;
                const float c1 = m_old[1] > -INFINITY ? exp2f(m_old[1] - m_r[1]) : 0.0f;
                l_r[0] *= c0; l_r[1] *= c1;
#pragma unroll
                for (int i = 0; i < HD / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
            }
            uint32_t pa[4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                float p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    p[e] = exp2f(sacc[nt][e] - m_r[e >> 1]);
                    l_r[e >> 1] += p[e];
                }
                pa[nt * 2 + 0] = pack_bf16(p[0], p[1]);
                pa[nt * 2 + 1] = pack_bf16(p[2], p[3]);
            }
            // O[16 heads][HD] += P[16][16] V[16][HD]
            const int key = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
            for (int np = 0; np < HD / 16; ++np) {
                const int dchunk = 2 * np + (lane >> 4);
                const uint32_t addr = vaddr + (uint32_t)((dchunk >> 3) * HALF_BYTES + key * 128 + (((dchunk & 7) ^ (key & 7)) << 4));
                uint32_t r0, r1, r2, r3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
                mma_bf16_16816(o[2 * np], pa, r0, r1);
                mma_bf16_16816(o[2 * np + 1], pa, r2, r3);
            }
        }
        __syncwarp();
        if (lane == 0)
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ring_smem(&bars[STAGES + s])) : "memory");
    }
    if (!ok && lane == 0 && a.status) atomicOr(a.status, MF_STATUS_WAIT_TIMEOUT);

    // the four lanes of a row each hold a part of its sum
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 1);
        l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 2);
    }
    if (t == 0) {
        ml_s[(warp * 16 + g) * 2 + 0] = m_r[0]; ml_s[(warp * 16 + g) * 2 + 1] = l_r[0];
        ml_s[(warp * 16 + g + 8) * 2 + 0] = m_r[1]; ml_s[(warp * 16 + g + 8) * 2 + 1] = l_r[1];
    }
    // consumers only (the producer has left): every warp is done with the ring
    asm volatile("bar.sync 1, %0;" ::"n"(RING_CONSUMERS * 32) : "memory");
    if (tid < 16) {
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < RING_CONSUMERS; ++w) m = fmaxf(m, ml_s[(w * 16 + tid) * 2]);
        float l = 0.0f;
#pragma unroll
        for (int w = 0; w < RING_CONSUMERS; ++w) {
            const float mw = ml_s[(w * 16 + tid) * 2];
            const float f = mw > -INFINITY ? exp2f(mw - m) : 0.0f;
            f_s[w * 16 + tid] = f;
            l += ml_s[(w * 16 + tid) * 2 + 1] * f;
        }
        l_s[tid] = l;
        if (tid < G && a.n_chunks > 1) {
            float* p = part0 + (size_t)tid * a.n_chunks * part_stride;
            p[0] = m * 0.6931471805599453f;           // back to natural-log units for the merge
            p[1] = l;
        }
    }
    float* ow = o_s + (size_t)warp * 16 * OS;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        *reinterpret_cast<float2*>(ow + (size_t)g * OS + nt * 8 + 2 * t) = make_float2(o[nt][0], o[nt][1]);
        if (G > 8)
            *reinterpret_cast<float2*>(ow + (size_t)(g + 8) * OS + nt * 8 + 2 * t) = make_float2(o[nt][2], o[nt][3]);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(RING_CONSUMERS * 32) : "memory");
    for (int idx = tid; idx < G * HD; idx += RING_CONSUMERS * 32) {
        const int r = idx / HD, d = idx - r * HD;
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < RING_CONSUMERS; ++w) acc = fmaf(o_s[((size_t)w * 16 + r) * OS + d], f_s[w * 16 + r], acc);
        if (a.n_chunks > 1)
            part0[(size_t)r * a.n_chunks * part_stride + 2 + d] = acc;
        else
            ((__nv_bfloat16*)a.out)[((size_t)row * a.n_heads + (size_t)hk * G + r) * HD + d] =
                __float2bfloat16(acc / l_s[r]);
    }
}

// ---- tensor maps over a layer's cache ----------------------------------------------------------
typedef CUresult (*RingEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static RingEncodeFn ring_encode_fn() {
    static RingEncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (RingEncodeFn)p;
    });
    return fn;
}

struct CacheMapKey {
    const void* ptr; long long rows; int hd;
    bool operator==(const CacheMapKey& o) const { return ptr == o.ptr && rows == o.rows && hd == o.hd; }
};
struct CacheMapKeyHash {
    size_t operator()(const CacheMapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ (size_t)k.rows * 1315423911u ^ (size_t)k.hd * 97u;
    }
};

// bfloat16 cache of a layer seen as [rows][hd]; a cache does not move, so its map is made once
static int cache_map(CUtensorMap* out, const void* ptr, long long rows, int hd) {
    static std::unordered_map<CacheMapKey, CUtensorMap, CacheMapKeyHash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const CacheMapKey key{ptr, rows, hd};
    auto it = cache.find(key);
    if (it == cache.end()) {
        RingEncodeFn fn = ring_encode_fn();
        if (!fn) return MF_ERR_NO_TENSORMAP;
        if (((uintptr_t)ptr & 15) != 0 || rows <= 0 || rows > 0x7fffffffLL) return MF_ERR_UNSUPPORTED;
        CUtensorMap m;
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
        cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
        cuuint32_t box[2] = {64, MF_PAGE};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return MF_ERR_TENSORMAP;
        it = cache.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}

template <int HD, int STAGES, int MINB>
static int launch_decode_ring(const AttnArgs& a, long long cache_rows, cudaStream_t stream) {
    constexpr int smem = 1024 + STAGES * 2 * (HD / 64) * MF_PAGE * 128 + 2 * STAGES * 8 +
                         RING_CONSUMERS * 16 * 3 * 4 + 16 * 4 + 16;
    static_assert(RING_CONSUMERS * 16 * (HD + 8) * 4 <= STAGES * 2 * (HD / 64) * MF_PAGE * 128,
                  "the warps' results fit over the ring");
    CUtensorMap mk, mv;
    if (int e = cache_map(&mk, a.k, cache_rows, HD)) return e;
    if (int e = cache_map(&mv, a.v, cache_rows, HD)) return e;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_ring_kernel<HD, STAGES, MINB>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(a.n_chunks, a.n_kv, a.rows);
    mf_launch(attention_decode_ring_kernel<HD, STAGES, MINB>, dim3(grid), dim3(RING_THREADS), smem, stream,
              mk, mv, a);
    return MF_LAUNCH_CHECK();
}

template <int HD>
static int launch_decode_mma(const AttnArgs& a, cudaStream_t stream) {
    // chunks of several blocks carry more state in registers: two CTAs per SM
    if (a.chunk > 256) return launch_decode_mma_as<HD, 2, true>(a, stream);
    const long long ctas = (long long)a.n_chunks * a.n_kv * a.rows;
    return ctas > 4 * mf_sm_count() ? launch_decode_mma_as<HD, 3, false>(a, stream)
                          : launch_decode_mma_as<HD, 2, false>(a, stream);
}

// MINFER_B200_DECODE_RING=0 keeps the kernel whose warps load their own keys (read once)
static int decode_ring_mode() {
    static int mode = -1;
    if (mode < 0) { const char* ev = getenv("MINFER_B200_DECODE_RING"); mode = ev ? atoi(ev) : 1; }
    return mode;
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
        mf_launch(attention_generic_kernel<float, false>, dim3(blocks), dim3(ATT_WARPS * 32), 0, stream, a);
    else if (dtype == MF_DTYPE_BF16)
        mf_launch(attention_generic_kernel<__nv_bfloat16, false>, dim3(blocks), dim3(ATT_WARPS * 32), 0, stream, a);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}

// Attention over the paged cache.  `partial` must hold rows*n_heads*n_chunks*(hd+2) floats
// when n_chunks > 1; chunk c covers absolute positions [c*chunk, (c+1)*chunk).  `cache_pages`
// (pages the cache tensors hold; 0 = unknown) and `status` (may be null) open the TMA-ring kernel.
// `old_keys_final`: every row is its sequence's only new token in this step, so the keys below
// its position were in the cache before the step began (the ring kernel then asks for them while
// the kernel before it still runs).
extern "C" int mf_attention_paged(const void* q, const void* k_cache, const void* v_cache,
                                  const int* row_seq, const int* row_pos, const int* page_table,
                                  int table_stride, int ring, void* out, float* partial, int rows,
                                  int n_heads, int n_kv, int hd, int window, int chunk, int n_chunks,
                                  float scale, int dtype, int force_generic, long long cache_pages,
                                  unsigned* status, int old_keys_final, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (int e = check_sizes(n_heads, n_kv, hd)) return e;
    if (n_chunks < 1 || (n_chunks > 1 && (partial == nullptr || chunk <= 0))) return MF_ERR_ARGUMENT;
    if (n_chunks > 6000) return MF_ERR_UNSUPPORTED;    // the merge keeps two floats per chunk in shared memory
    if (ring % MF_PAGE != 0) return MF_ERR_ARGUMENT;
    AttnArgs a{};
    a.q = q; a.k = k_cache; a.v = v_cache; a.row_seq = row_seq; a.row_pos = row_pos;
    a.page_table = page_table; a.table_stride = table_stride; a.ring = ring;
    a.out = out; a.partial = n_chunks > 1 ? partial : nullptr;
    a.rows = rows; a.n_heads = n_heads; a.n_kv = n_kv; a.hd = hd; a.window = window;
    a.chunk = chunk; a.n_chunks = n_chunks; a.scale = scale;
    // tensor-core path: bfloat16, head size 64 or 128, groups of up to 16 heads, 256-key chunks
    const bool fast = dtype == MF_DTYPE_BF16 && (hd == 64 || hd == 128) && n_heads / n_kv <= 16 &&
                      chunk >= 256 && chunk % 256 == 0 && partial != nullptr && rows <= 65535 && n_kv <= 65535 &&
                      !force_generic;
    if (fast) {
        a.partial = partial;
        a.status = status;
        a.old_keys_final = old_keys_final;
        // the TMA ring needs the cache's extent for its tensor maps and a status word for its
        // bounded waits; without them, or with MINFER_B200_DECODE_RING=0, the kernel whose warps
        // load their own keys runs (measured, 64 sequences at 2,048 positions: 44.5 against
        // 60.7 us; 8 at 8,192: 30.4 against 37.4; equal on chunks of a single block)
        const int ring_mode = decode_ring_mode();
        int e;
        if (ring_mode && cache_pages > 0 && status != nullptr) {
            const long long cache_rows = cache_pages * n_kv * MF_PAGE;
            e = hd == 64 ? launch_decode_ring<64, 6, 2>(a, cache_rows, stream)
                         : launch_decode_ring<128, 3, 2>(a, cache_rows, stream);
        } else {
            e = hd == 64 ? launch_decode_mma<64>(a, stream) : launch_decode_mma<128>(a, stream);
        }
        if (e || n_chunks == 1) return e;
        // measured: started early, the merge of the chunks costs 5 us more than it saves (its
        // blocks sit on the SMs while the last attention blocks still look for room); the same
        // with the ring kernel and all CTAs resident at once (3.25 against 3.16 ms a step).
        // Seen on the step's timeline: started early, the output projection behind it gets on
        // the SMs 4 us sooner and has its weights by the time the merge ends (8.3 -> 4.4 us),
        // but those 26 MB share HBM with the keys (attention 7.1 -> 8.2 us, merge 3.3 -> 4.8)
        mf_launch_ex(false, attention_combine_kernel<__nv_bfloat16>, dim3(rows * n_heads), dim3(hd),
                     (size_t)n_chunks * 8, stream, partial, (__nv_bfloat16*)out, n_chunks, hd);
        return MF_LAUNCH_CHECK();
    }
    const long long items = (long long)rows * n_heads * n_chunks;
    const unsigned blocks = (unsigned)((items + ATT_WARPS - 1) / ATT_WARPS);
    if (dtype == MF_DTYPE_F32)
        mf_launch(attention_generic_kernel<float, true>, dim3(blocks), dim3(ATT_WARPS * 32), 0, stream, a);
    else if (dtype == MF_DTYPE_BF16)
        mf_launch(attention_generic_kernel<__nv_bfloat16, true>, dim3(blocks), dim3(ATT_WARPS * 32), 0, stream, a);
    else
        return MF_ERR_UNSUPPORTED;
    int e = MF_LAUNCH_CHECK();
    if (e || n_chunks == 1) return e;
    const int threads = hd >= 128 ? 128 : (hd >= 64 ? 64 : 32);
    if (dtype == MF_DTYPE_F32)
        mf_launch(attention_combine_kernel<float>, dim3(rows * n_heads), dim3(threads), (size_t)n_chunks * 8, stream,
            partial, (float*)out, n_chunks, hd);
    else
        mf_launch(attention_combine_kernel<__nv_bfloat16>, dim3(rows * n_heads), dim3(threads), (size_t)n_chunks * 8, stream,
            partial, (__nv_bfloat16*)out, n_chunks, hd);
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// The same attention for callers that cannot allocate device memory (see
// attention_noalloc.h for who they are and for the limits).  The scratch that merges key
// chunks lives in this fixed array.  In host code the array's name only stands for the
// symbol: it is not a device address, so the address is looked up once per device and that
// pointer is what the kernels get.
// ------------------------------------------------------------------------------------------
#include "attention_noalloc.h"

static __device__ __align__(256) float mf_noalloc_scratch[MF_ATTENTION_NOALLOC_FLOATS];

static float* noalloc_scratch_of_device[MF_MAX_DEVICES];

extern "C" long long mf_attention_noalloc_capacity(void) {
    return (long long)MF_ATTENTION_NOALLOC_FLOATS;
}

extern "C" int mf_attention_paged_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                          const int* row_seq, const int* row_pos,
                                          const int* page_table, int table_stride, int ring,
                                          void* out, int rows, int n_heads, int n_kv, int hd,
                                          int window, int chunk, int n_chunks, float scale,
                                          int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n_chunks < 1) return MF_ERR_ARGUMENT;
    if (int bad = check_sizes(n_heads, n_kv, hd)) return bad;
    // every factor is checked against the array before it is multiplied in: no overflow
    const long long cap = (long long)MF_ATTENTION_NOALLOC_FLOATS;
    long long need = (long long)hd + 2;
    const int factors[3] = {rows, n_heads, n_chunks};
    for (int f : factors) {
        if ((long long)f > cap) return MF_ERR_SCRATCH_LIMIT;
        need *= f;
        if (need > cap) return MF_ERR_SCRATCH_LIMIT;
    }
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= MF_MAX_DEVICES) return MF_ERR_UNSUPPORTED;
    if (noalloc_scratch_of_device[device] == nullptr) {
        // set-up, once per device, with that device current: the array's address, the shared
        // memory of every kernel variant a later call may pick, and the environment switch.
        // (Two host threads that make their first calls at once both do this and store the
        // same values: harmless.)
        float* address = nullptr;
        e = cudaGetSymbolAddress((void**)&address, mf_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (int bad = configure_decode_mma_all()) return bad;
        (void)decode_ring_mode();
        noalloc_scratch_of_device[device] = address;
    }
    return mf_attention_paged(q, k_cache, v_cache, row_seq, row_pos, page_table, table_stride, ring,
                              out, noalloc_scratch_of_device[device], rows, n_heads, n_kv, hd, window,
                              chunk, n_chunks, scale, dtype, 0, 0, nullptr, 0, stream);
}
