// Attention of whole prompts on the 5th-generation tensor cores (bfloat16, head size 64 or 128):
// causal, grouped query heads, optional window, sequences of unequal lengths packed one after
// another.  Same formula as the other attention kernels (src/graph/cpu_backend.rs:437-494 in
// the reference): scores * scale, mask by position, softmax in float32, weighted sum of values.
//
// A CTA owns 256 queries of one head as two tiles of 128 and walks the keys in tiles of 128;
// both query tiles use every key tile, so keys and values cross L2 -> shared memory once for
// 256 queries (one query tile per CTA was bound by that traffic):
//   S = Q K^T     tcgen05.mma, both operands in shared memory (TMA, 128-byte swizzle), S in
//                 tensor memory, one S buffer for each query tile
//   softmax       one warpgroup for each query tile, one thread per query row: the row of S
//                 comes out of tensor memory into registers once, maximum / exp2 / sum in
//                 float32, and the probabilities go back into the same columns as packed
//                 bfloat16.  The two warpgroups take their registers from the first one
//                 (setmaxnreg), which only issues copies and MMAs
//   O += P V      tcgen05.mma with P read from tensor memory as the A operand and V from
//                 shared memory as an MN-major B operand; O stays in tensor memory (one for
//                 each query tile) and is rescaled there by the softmax threads only when a
//                 row's maximum has grown
//   The MMA thread alternates between the query tiles: O += P V of a key tile as soon as
//   its probabilities are there, then at once S of the next key tile into the same columns;
//   while one query tile is in its softmax the tensor cores work for the other.
//   Tensor memory: S0 S1 O0 O1 = 512 columns.  Shared memory: Q 2 tiles, K and V rings of 2.
//   warp 0: TMA producer; warp 1: MMA issuer; warps 4-7 and 8-11: softmax and the final
//   O / sum of query tile 0 and 1.  The second tile may lie beyond the sequence (or see other
//   key tiles than the first: causal edge, window): each tile has its own range of key tiles.
// Rows of the packed tensors that lie beyond a sequence's end belong to the next sequence;
// they are masked by position, never used.  Every mbarrier wait is bounded.
//
// PAGED: the step's tokens go on from what the cache holds (a prompt's later portion, several
// tokens onto a sequence, rows that start beside rows that go on).  The queries are the
// step's packed rows as before, at absolute positions start + i with start = the sequence's
// length before the step; keys and values are read from the paged cache, which holds the
// step's own by then (the kernel before this one wrote them).  A key tile is 128 absolute
// positions = two pages of one key/value head, fetched as two boxes of 64 rows through tensor
// maps over the layer's cache; the mask is by absolute position.  Positions of a page beyond a
// sequence's end hold finite leftovers (storage is zeroed once and only ever written by
// kernels); causality masks them.
#include <cuda.h>

#include "common.cuh"

#define FA_Q 128              // queries per tile
#define FA_CTA_Q 256          // a CTA owns two query tiles that share every key tile
#define FA_KEYS 128           // keys per tile
#define FA_LAZY_LOG2 8.0f      // the maximum may grow this many binary orders before O is rescaled
#define FA_THREADS 384        // warp 0 TMA, warp 1 MMA, warps 4-7 and 8-11 softmax of the two query tiles
#define FA_MAX_SPIN (1u << 24)
#define FA_MAX_WAIT_NS 2000000000ull

#define MF_ERR_NO_TENSORMAP 2003
#define MF_ERR_TENSORMAP 2004

struct FaArgs {
    const int* cu_seqlens;
    __nv_bfloat16* out;       // [tokens][n_heads * HD]
    unsigned* status;
    int n_heads, n_kv, window;
    float scale_log2;         // scale * log2(e)
    // PAGED only
    const int* seq_end;       // [sequences] length after this step
    const int* page_table;    // [sequences][table_stride] pages of 64 positions, -1 = none
    int table_stride;
    int ring;                 // 0 = linear, else position p lies at p % ring
};

// ---- PTX wrappers --------------------------------------------------------------------------
__device__ __forceinline__ uint32_t fa_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fa_bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fa_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fa_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool fa_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool fa_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it < FA_MAX_SPIN; ++it) {
        if (fa_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if ((it & 1023u) == 1023u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > FA_MAX_WAIT_NS) break;
        }
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void fa_tma(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void fa_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fa_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fa_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void fa_mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void fa_mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
        ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void fa_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void fa_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void fa_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void fa_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fa_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// K-major operand tile whose rows are 128 bytes (64 bf16), 128-byte swizzle: 8-row groups
// 1024 bytes apart.
__device__ __forceinline__ uint64_t fa_desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand (the values: rows are keys = the K dimension, 64 head dimensions = 128
// bytes per row, 128-byte swizzle): the next 64 head dimensions lie `lbo` bytes further
// (leading offset), 8-key groups 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t fa_desc_mnmajor(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// Two float32 in one 64-bit register, and the packed forms of fma and add (each half is the
// scalar operation, round to nearest), and the maximum of three.
__device__ __forceinline__ uint64_t fa_pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void fa_unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fa_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t fa_add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float fa_max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ uint32_t fa_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD, bool PAGED>
__global__ void __launch_bounds__(FA_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const FaArgs a) {
    pdl_prologue();
    constexpr int NB = HD / 64;                         // 64-column blocks per row
    constexpr int BLOCK = 128 * 128;                    // bytes of a [128 rows][64 cols] block
    constexpr int T_BYTES = NB * BLOCK;                 // a [128 rows][HD] tile
    constexpr int TM_S = 0, TM_O = 256;                 // tensor memory columns; tile t: + 128 t
    extern __shared__ uint8_t fa_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)fa_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;                                // [2 query tiles][NB][128][64]
    uint8_t* k_s = q_s + 2 * T_BYTES;                   // [2 stages]
    uint8_t* v_s = k_s + 2 * T_BYTES;                   // [2 stages]
    uint64_t* bars = (uint64_t*)(v_s + 2 * T_BYTES);
    uint64_t* q_full = bars;                            // 1
    uint64_t* k_full = bars + 1;                        // [2 stages]
    uint64_t* k_empty = bars + 3;
    uint64_t* v_full = bars + 5;
    uint64_t* v_empty = bars + 7;
    uint64_t* s_full = bars + 9;                        // [2 query tiles]
    uint64_t* p_full = bars + 11;                       // [2 query tiles], 128 arrivals
    uint64_t* o_done = bars + 13;                       // [2 query tiles]
    uint32_t* tmem_slot = (uint32_t*)(bars + 15);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = blockIdx.z, head = blockIdx.x;
    const int tok0 = a.cu_seqlens[seq];
    const int len = a.cu_seqlens[seq + 1] - tok0;
    const int q0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * FA_CTA_Q;     // heavy tiles first
    if (q0 >= len) return;
    const int hk = head / (a.n_heads / a.n_kv);
    // position of the step's first token of this sequence (0 for whole prompts), and the end of
    // the keys that exist: packed keys end with the sequence, cached ones are masked by causality
    const int pos0 = PAGED ? a.seq_end[seq] - len : 0;
    const int key_end = PAGED ? 0x7fffffff : len;
    // the key tiles of each query tile: [kb, ke); the second tile may be beyond the sequence
    int kb[2], ke[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int q0t = q0 + t * FA_Q;
        if (q0t < len) {
            kb[t] = a.window > 0 ? max(0, pos0 + q0t - a.window + 1) / FA_KEYS : 0;
            ke[t] = (pos0 + min(q0t + FA_Q, len) - 1) / FA_KEYS + 1;
        } else {
            kb[t] = ke[t] = 0;
        }
    }
    const bool has1 = ke[1] > kb[1];
    const int lo = kb[0], hi = has1 ? ke[1] : ke[0];
    const int n_tiles = hi - lo;

    if (tid == 0) {
        fa_bar_init(fa_smem(q_full), 1);
        for (int i = 0; i < 2; ++i) {
            fa_bar_init(fa_smem(&k_full[i]), 1);
            fa_bar_init(fa_smem(&k_empty[i]), 1);
            fa_bar_init(fa_smem(&v_full[i]), 1);
            fa_bar_init(fa_smem(&v_empty[i]), 1);
            fa_bar_init(fa_smem(&s_full[i]), 1);
            fa_bar_init(fa_smem(&p_full[i]), 128);
            fa_bar_init(fa_smem(&o_done[i]), 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(fa_smem(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fa_fence_before();
    __syncthreads();
    fa_fence_after();
    const uint32_t tmem = *tmem_slot;

    // Registers: the kernel is compiled for 168 a thread (three warps on a scheduler); the first
    // warpgroup gives most of its share back and the softmax warpgroups, which hold a whole
    // row of scores each, take it.
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
      if (warp == 0 && lane == 0) {
        // ---- TMA producer ---------------------------------------------------------------
        fa_expect_tx(fa_smem(q_full), has1 ? 2 * T_BYTES : T_BYTES);
        for (int t = 0; t < (has1 ? 2 : 1); ++t)
            for (int c = 0; c < NB; ++c)
                fa_tma(fa_smem(q_s + t * T_BYTES + c * BLOCK), &map_q, head * HD + 64 * c,
                       tok0 + q0 + t * FA_Q, fa_smem(q_full));
        for (int i = 0; i < n_tiles; ++i) {
            const int st = i & 1;
            const uint32_t free_parity = (uint32_t)((i >> 1) & 1) ^ 1u;
            if (PAGED) {
                // the tile's two pages: rows (page * n_kv + hk) * 64 .. + 63 of the cache seen as
                // [rows][HD]; a page the sequence does not have (beyond its end) reads page 0,
                // whose positions causality masks
                int y[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int p = (lo + i) * FA_KEYS + h * MF_PAGE;
                    const int idx = (a.ring > 0 ? p % a.ring : p) >> 6;
                    int page = idx < a.table_stride ? a.page_table[(size_t)seq * a.table_stride + idx] : 0;
                    if (page < 0) page = 0;
                    y[h] = (page * a.n_kv + hk) * MF_PAGE;
                }
                if (!fa_wait(fa_smem(&k_empty[st]), free_parity, abort_flag)) break;
                fa_expect_tx(fa_smem(&k_full[st]), T_BYTES);
                for (int c = 0; c < NB; ++c)
                    for (int h = 0; h < 2; ++h)
                        fa_tma(fa_smem(k_s + st * T_BYTES + c * BLOCK + h * (BLOCK / 2)), &map_k, 64 * c, y[h],
                               fa_smem(&k_full[st]));
                if (!fa_wait(fa_smem(&v_empty[st]), free_parity, abort_flag)) break;
                fa_expect_tx(fa_smem(&v_full[st]), T_BYTES);
                for (int c = 0; c < NB; ++c)
                    for (int h = 0; h < 2; ++h)
                        fa_tma(fa_smem(v_s + st * T_BYTES + c * BLOCK + h * (BLOCK / 2)), &map_v, 64 * c, y[h],
                               fa_smem(&v_full[st]));
                continue;
            }
            const int key0 = tok0 + (lo + i) * FA_KEYS;
            if (!fa_wait(fa_smem(&k_empty[st]), free_parity, abort_flag)) break;
            fa_expect_tx(fa_smem(&k_full[st]), T_BYTES);
            for (int c = 0; c < NB; ++c)
                fa_tma(fa_smem(k_s + st * T_BYTES + c * BLOCK), &map_k, hk * HD + 64 * c, key0,
                       fa_smem(&k_full[st]));
            if (!fa_wait(fa_smem(&v_empty[st]), free_parity, abort_flag)) break;
            fa_expect_tx(fa_smem(&v_full[st]), T_BYTES);
            for (int c = 0; c < NB; ++c)
                fa_tma(fa_smem(v_s + st * T_BYTES + c * BLOCK), &map_v, hk * HD + 64 * c, key0,
                       fa_smem(&v_full[st]));
        }
      } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer -------------------------------------------------------------------
        // S: M = 128 queries, N = 128 keys, both operands K-major
        constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(FA_KEYS >> 3) << 17) |
                                     ((uint32_t)(128 >> 4) << 24);
        // O: M = 128 queries, N = HD, A from tensor memory, B MN-major
        constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                     ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        auto issue_qk = [&](int t, int i) {
            const uint32_t q_addr = fa_smem(q_s + t * T_BYTES);
            const uint32_t k_addr = fa_smem(k_s + (i & 1) * T_BYTES);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                const uint32_t off = (uint32_t)((ks >> 2) * BLOCK + (ks & 3) * 32);
                fa_mma_ss(tmem + (uint32_t)(TM_S + t * 128), fa_desc_kmajor(q_addr + off),
                          fa_desc_kmajor(k_addr + off), idesc_s, ks > 0 ? 1u : 0u);
            }
            fa_commit(fa_smem(&s_full[t]));
        };
        int done[2] = {0, 0};                            // products P V issued for each query tile
        bool ok = fa_wait(fa_smem(q_full), 0u, abort_flag);
        if (ok) ok = fa_wait(fa_smem(&k_full[0]), 0u, abort_flag);
        if (ok) {
            fa_fence_after();
#pragma unroll
            for (int t = 0; t < 2; ++t)
                if (lo >= kb[t] && lo < ke[t]) issue_qk(t, 0);
            fa_commit(fa_smem(&k_empty[0]));
        }
        // per key tile and query tile: O += P V for this key tile as soon as its probabilities
        // are there, then at once S = Q K^T for the next key tile into the same columns; while
        // one query tile is in its softmax the tensor cores work for the other
        for (int i = 0; i < n_tiles && ok; ++i) {
            const int j = lo + i;
            const bool next = i + 1 < n_tiles;
            ok = fa_wait(fa_smem(&v_full[i & 1]), (uint32_t)((i >> 1) & 1), abort_flag);
            if (ok && next) ok = fa_wait(fa_smem(&k_full[(i + 1) & 1]), (uint32_t)(((i + 1) >> 1) & 1), abort_flag);
            if (!ok) break;
            fa_fence_after();
            const uint32_t v_addr = fa_smem(v_s + (i & 1) * T_BYTES);
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const bool cur = j >= kb[t] && j < ke[t];
                const bool nxt = next && j + 1 >= kb[t] && j + 1 < ke[t];
                if (cur) {
                    ok = fa_wait(fa_smem(&p_full[t]), (uint32_t)(done[t] & 1), abort_flag);
                    if (!ok) break;
                    fa_fence_after();
#pragma unroll
                    for (int ks = 0; ks < FA_KEYS / 16; ++ks)
                        fa_mma_ts(tmem + (uint32_t)(TM_O + t * 128), tmem + (uint32_t)(TM_S + t * 128 + ks * 8),
                                  fa_desc_mnmajor(v_addr + (uint32_t)(ks * 16 * 128), BLOCK), idesc_o,
                                  (done[t] > 0 || ks > 0) ? 1u : 0u);
                    ++done[t];
                }
                if (nxt) issue_qk(t, i + 1);
                else if (cur) fa_commit(fa_smem(&o_done[t]));
            }
            if (!ok) break;
            fa_commit(fa_smem(&v_empty[i & 1]));
            if (next) fa_commit(fa_smem(&k_empty[(i + 1) & 1]));
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        // ---- softmax: four warps for each query tile, one thread per query row ----------------
        const int t = (warp - 4) >> 2;
        const int quarter = warp & 3;                    // the 32 TMEM lanes this warp may touch
        const int row = quarter * 32 + lane;             // row of the tile = TMEM lane
        const int q0t = q0 + t * FA_Q;
        const int qrow = q0t + row;                      // this thread's query among the sequence's rows
        const int qpos = pos0 + qrow;                    // and its absolute position
        const int wpos = pos0 + q0t + quarter * 32;      // position of this warp's first query
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        const uint32_t s_addr = lane_addr + (uint32_t)(TM_S + t * 128);
        const uint32_t o_addr = lane_addr + (uint32_t)(TM_O + t * 128);
        const int kb_t = t ? kb[1] : kb[0], ke_t = t ? ke[1] : ke[0];
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = kb_t; j < ke_t; ++j) {
            const int c = j - kb_t;
            const int key0 = j * FA_KEYS;
            // S of this key tile is complete, and with it every earlier product of this query tile
            if (!fa_wait(fa_smem(&s_full[t]), (uint32_t)(c & 1), abort_flag)) { ok = false; break; }
            fa_fence_after();
            const bool need_mask = key0 + FA_KEYS - 1 > wpos || key0 + FA_KEYS > key_end ||
                                   (a.window > 0 && key0 < wpos + 31 - a.window + 1);
            // the whole row of S (128 scores) into registers, masked by position where the tile
            // touches the diagonal, the window's edge or the sequence's end
            uint32_t sr[FA_KEYS];
#pragma unroll
            for (int c0 = 0; c0 < FA_KEYS; c0 += 32) fa_ld32(s_addr + (uint32_t)c0, sr + c0);
            fa_wait_ld();
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < FA_KEYS; ++i) {
                    const int key = key0 + i;
                    const bool vis = key <= qpos && key < key_end && (a.window == 0 || qpos - key < a.window);
                    if (!vis) sr[i] = 0xff800000u;            // -inf
                }
            }
            // the maximum with four independent chains of three-input maxima
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < FA_KEYS; i += 8) {
                mx0 = fa_max3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
                mx1 = fa_max3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
                mx2 = fa_max3(mx2, __uint_as_float(sr[i + 4]), __uint_as_float(sr[i + 5]));
                mx3 = fa_max3(mx3, __uint_as_float(sr[i + 6]), __uint_as_float(sr[i + 7]));
            }
            const float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            // The reference point of the exponentials moves only when the maximum has grown by more
            // than FA_LAZY_LOG2 binary orders (softmax does not depend on the point; until then a
            // probability is at most 2^FA_LAZY_LOG2 before the division by the sum, far inside
            // float32 and bfloat16).  The output so far has to be rescaled when the point moves,
            // a round trip of 128 columns through tensor memory in the middle of the softmax.
            const bool jump = m == -INFINITY ? m_tile > -INFINITY
                                             : (m_tile - m) * a.scale_log2 > FA_LAZY_LOG2;
            const float m_new = jump ? m_tile : m;
            const float m_off = m_new == -INFINITY ? 0.0f : m_new * a.scale_log2;
            const float corr = m == -INFINITY ? 0.0f : exp2f(m * a.scale_log2 - m_off);
            // the output so far is rescaled only if the point moved for some row of this warp
            const bool grow = m_new > m;
            if (c > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t r[32];
                    fa_ld32(o_addr + (uint32_t)c0, r);
                    fa_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
                    fa_st32(o_addr + (uint32_t)c0, r);
                }
            }
            m = m_new;
            // probabilities (ex2.approx of the scaled difference), their sum with four chains,
            // packed as bfloat16 pairs into the first 64 columns of this S buffer
            // (two scores an instruction: the scaled differences and the sums are packed pairs of
            // float32, the same operations on each half as the scalar forms)
            uint64_t l01 = 0, l23 = 0;                   // {l0, l1}, {l2, l3} = four zeros
            const uint64_t scale2 = fa_pack2(a.scale_log2, a.scale_log2), off2 = fa_pack2(-m_off, -m_off);
            uint32_t pk[FA_KEYS / 2];
#pragma unroll
            for (int i = 0; i < FA_KEYS; i += 4) {
                float x0, x1, x2, x3, p0, p1, p2, p3;
                fa_unpack2(fa_fma2(fa_pack2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), scale2, off2), x0, x1);
                fa_unpack2(fa_fma2(fa_pack2(__uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3])), scale2, off2), x2, x3);
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(x0));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(x1));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p2) : "f"(x2));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p3) : "f"(x3));
                l01 = fa_add2(l01, fa_pack2(p0, p1));
                l23 = fa_add2(l23, fa_pack2(p2, p3));
                pk[i >> 1] = fa_pack(p0, p1);
                pk[(i >> 1) + 1] = fa_pack(p2, p3);
            }
            float l0, l1, l2, l3;
            fa_unpack2(l01, l0, l1);
            fa_unpack2(l23, l2, l3);
            l = l * corr + ((l0 + l1) + (l2 + l3));
#pragma unroll
            for (int c0 = 0; c0 < FA_KEYS / 2; c0 += 32) fa_st32(s_addr + (uint32_t)c0, pk + c0);
            fa_wait_st();
            fa_fence_before();
            fa_arrive(fa_smem(&p_full[t]));
        }
        // ---- the result: O / sum -------------------------------------------------------------
        if (ok && ke_t > kb_t && fa_wait(fa_smem(&o_done[t]), 0u, abort_flag)) {
            fa_fence_after();
            const float inv = 1.0f / l;
            __nv_bfloat16* o = a.out + ((long long)(tok0 + qrow) * a.n_heads + head) * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t r[32];
                fa_ld32(o_addr + (uint32_t)c0, r);
                fa_wait_ld();
                if (qrow < len) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 v;
                        v.x = fa_pack(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                        v.y = fa_pack(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                        v.z = fa_pack(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
                        v.w = fa_pack(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(o + c0 + i) = v;
                    }
                }
            }
        }
    }
    __syncwarp();
    fa_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0) {
        atomicOr(a.status, MF_STATUS_WAIT_TIMEOUT);
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*FaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);

static FaEncodeFn fa_encode_fn() {
    static FaEncodeFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (FaEncodeFn)p;
    }
    return fn;
}

// [tokens][width] bf16, box = [128 rows][64 columns]
static int fa_map(CUtensorMap* map, const void* ptr, long long tokens, long long width) {
    FaEncodeFn fn = fa_encode_fn();
    if (!fn) return MF_ERR_NO_TENSORMAP;
    cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)tokens};
    cuuint64_t strides[1] = {(cuuint64_t)width * 2};
    cuuint32_t box[2] = {64, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : MF_ERR_TENSORMAP;
}

// the paged cache of a layer seen as [rows][hd] bf16, box = one page of one key/value head as
// [64 rows][64 columns]
static int fa_cache_map(CUtensorMap* map, const void* ptr, long long rows, int hd) {
    FaEncodeFn fn = fa_encode_fn();
    if (!fn) return MF_ERR_NO_TENSORMAP;
    if (rows <= 0 || rows > 0x7fffffffLL) return MF_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, MF_PAGE};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : MF_ERR_TENSORMAP;
}

template <int HD, bool PAGED>
static int fa_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FaArgs& a,
                     int n_seqs, int max_len, cudaStream_t stream) {
    constexpr int smem = (HD / 64) * 16384 * 6 + 1024 + 256;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD, PAGED>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(a.n_heads, (max_len + FA_CTA_Q - 1) / FA_CTA_Q, n_seqs);
    mf_launch(attention_prefill_tc_kernel<HD, PAGED>, grid, dim3(FA_THREADS), smem, stream, mq, mk, mv, a);
    return MF_LAUNCH_CHECK();
}

// q [tokens][n_heads][hd], k/v [tokens][n_kv][hd], out [tokens][n_heads*hd], all bfloat16 and
// contiguous; sequence b holds tokens cu_seqlens[b] .. cu_seqlens[b+1]-1 at positions 0, 1, ...
extern "C" int mf_attention_prefill_tc(const void* q, const void* k, const void* v, const int* cu_seqlens,
                                       void* out, int n_tokens, int n_seqs, int max_len, int n_heads,
                                       int n_kv, int hd, int window, float scale, unsigned* status,
                                       cudaStream_t stream) {
    if (n_seqs <= 0 || max_len <= 0 || n_tokens <= 0) return 0;
    if ((hd != 64 && hd != 128) || n_kv <= 0 || n_heads % n_kv != 0) return MF_ERR_UNSUPPORTED;
    if (n_seqs > 65535 || (max_len + FA_CTA_Q - 1) / FA_CTA_Q > 65535) return MF_ERR_UNSUPPORTED;
    if (((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15) || ((uintptr_t)out & 15))
        return MF_ERR_UNSUPPORTED;
    CUtensorMap mq, mk, mv;
    if (int e = fa_map(&mq, q, n_tokens, (long long)n_heads * hd)) return e;
    if (int e = fa_map(&mk, k, n_tokens, (long long)n_kv * hd)) return e;
    if (int e = fa_map(&mv, v, n_tokens, (long long)n_kv * hd)) return e;
    FaArgs a{};
    a.cu_seqlens = cu_seqlens; a.out = (__nv_bfloat16*)out; a.status = status;
    a.n_heads = n_heads; a.n_kv = n_kv; a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    return hd == 64 ? fa_launch<64, false>(mq, mk, mv, a, n_seqs, max_len, stream)
                    : fa_launch<128, false>(mq, mk, mv, a, n_seqs, max_len, stream);
}

// The step's tokens (q [tokens][n_heads][hd], sequence b = tokens cu_seqlens[b] .. cu_seqlens[b+1]-1,
// max_len the most of one sequence) at positions seq_end[b] - count .. seq_end[b] - 1 attend over
// the paged cache k/v [cache_pages][n_kv][64][hd], which already holds those positions' own keys.
extern "C" int mf_attention_prefill_tc_paged(const void* q, const void* k_cache, const void* v_cache,
                                             const int* cu_seqlens, const int* seq_end, const int* page_table,
                                             int table_stride, int ring, void* out, int n_tokens, int n_seqs,
                                             int max_len, int n_heads, int n_kv, int hd, int window,
                                             float scale, long long cache_pages, unsigned* status,
                                             cudaStream_t stream) {
    if (n_seqs <= 0 || max_len <= 0 || n_tokens <= 0) return 0;
    if ((hd != 64 && hd != 128) || n_kv <= 0 || n_heads % n_kv != 0) return MF_ERR_UNSUPPORTED;
    if (n_seqs > 65535 || (max_len + FA_CTA_Q - 1) / FA_CTA_Q > 65535) return MF_ERR_UNSUPPORTED;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)out & 15))
        return MF_ERR_UNSUPPORTED;
    if (cache_pages <= 0 || table_stride <= 0 || ring % MF_PAGE != 0 || !seq_end || !page_table)
        return MF_ERR_ARGUMENT;
    CUtensorMap mq, mk, mv;
    if (int e = fa_map(&mq, q, n_tokens, (long long)n_heads * hd)) return e;
    if (int e = fa_cache_map(&mk, k_cache, cache_pages * n_kv * MF_PAGE, hd)) return e;
    if (int e = fa_cache_map(&mv, v_cache, cache_pages * n_kv * MF_PAGE, hd)) return e;
    FaArgs a{};
    a.cu_seqlens = cu_seqlens; a.out = (__nv_bfloat16*)out; a.status = status;
    a.n_heads = n_heads; a.n_kv = n_kv; a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.seq_end = seq_end; a.page_table = page_table; a.table_stride = table_stride; a.ring = ring;
    return hd == 64 ? fa_launch<64, true>(mq, mk, mv, a, n_seqs, max_len, stream)
                    : fa_launch<128, true>(mq, mk, mv, a, n_seqs, max_len, stream);
}
