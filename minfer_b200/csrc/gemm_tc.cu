// bfloat16 projections on the 5th-generation tensor cores:
//     Y[tokens][N] (+)= X[tokens][K] * W[N][K]^T (+ bias)
// tcgen05.mma with the accumulator in tensor memory, both operands staged in shared
// memory by TMA (128-byte swizzle), an mbarrier ring between the TMA thread, the MMA
// thread and the epilogue warps.  The reference multiplies with scalar SIMT kernels that
// re-read the weights for every token (src/cuda_kernels.cu:32-93, grid.y = tokens); here a
// weight tile is read once per step and the same kernel serves whole prompts (256-token
// tiles) and decoding (16..64-token tiles that stream the weights at memory speed).
//
// Roles of the operands are swapped against the usual convention: the WEIGHT tile
// [128 rows of W][64 k] is the MMA's M side, the token tile [NT tokens][64 k] its N side,
// so the accumulator holds D[n][token] with n along the 128 TMEM lanes.  A thread of the
// epilogue owns one n and walks over the tokens; a warp's store for one token covers 32
// consecutive n.
//
// Work that does not fill the GPU is split along K: each split writes float32 partial sums
// that mf_splitk_reduce adds in split order (no atomics, so results are reproducible).
//
// A norm between two products need not be a kernel of its own.  The product that completes the
// residual stream (EPI_ACCUM with `prep_x` set) also writes, for the norm that reads it next,
// x' = bfloat16(h * g) (g: that norm's weight) and, per group of output columns, the sum of h^2
// of every token (`prep_ssq`).  The product that follows takes x' as its token operand and
// multiplies token t's accumulators by 1 / sqrt(sum_parts ssq[.][t] / width + eps) in its
// epilogue (`row_ssq`): the same numbers as norm, then product, up to the place of one
// rounding.  This is done for few tokens (decoding), where a norm as a kernel of its own is a
// link in a chain of dependent launches: there the product that completes the residual is split
// along K over a CLUSTER of CTAs, which add their partial tiles in rank order through
// distributed shared memory (no atomics: reproducible), each finishing some of the tokens.
//
// Every wait on an mbarrier is bounded: when it runs out the kernel sets
// MF_STATUS_WAIT_TIMEOUT in the status word, stops issuing work, lets its copies land,
// frees its tensor memory and returns.
#include <cuda.h>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

#define TILE_N 128            // rows of W per CTA (MMA M)
#define TILE_K 64             // k per stage: 64 bf16 = 128 bytes = one swizzle row
#define A_BYTES (TILE_N * TILE_K * 2)
#define MAX_SPIN (1u << 24)
#define MAX_WAIT_NS 2000000000ull   // two seconds

#define EPI_STORE 0           // out = acc + bias          (float32 or bfloat16)
#define EPI_ACCUM 1           // out += acc + bias         (float32)
#define EPI_SWIGLU 2          // rows of W interleaved gate,up: out[j] = silu(g) * u (bfloat16)
#define EPI_PARTIAL 3         // ws[split][token][n] = acc (float32)

#define MF_ERR_NO_TENSORMAP 2003
#define MF_ERR_TENSORMAP 2004

struct GemmArgs {
    void* out;                // EPI_STORE/ACCUM/SWIGLU
    float* partial;           // EPI_PARTIAL
    const float* bias;
    unsigned* status;
    long long ldo;            // elements between consecutive tokens of out
    int M, N, K;              // tokens, rows of W, reduction length
    int kblocks_per_split;
    int epi;
    int out_dtype;
    // this product's token rows are x' = h * g of a norm whose 1/rms is still to be applied:
    // scale[t] = rsqrt(sum_{p < ssq_parts} row_ssq[p * M + t] / ssq_width + ssq_eps); null = none
    const float* row_ssq;
    int ssq_parts, ssq_width;
    float ssq_eps;
    // EPI_ACCUM only, null = none: after out[t][n] += acc, prep_x[t][n] = bfloat16(out[t][n] * prep_g[n])
    // and prep_ssq[part][t] = sum over the part's columns of out[t][n]^2
    __nv_bfloat16* prep_x;
    const float* prep_g;
    float* prep_ssq;
    long long ldp;            // elements between consecutive tokens of prep_x
};

// 1 / rms of the token rows m0 + t, t = first, first + step, .. < n_tok, into out[t] (shared
// memory): a thread adds a token's parts in order, all of its loads in flight together.
__device__ __forceinline__ void row_scales(const GemmArgs& a, int m0, int n_tok, float* out, int first, int step) {
    for (int t = first; t < n_tok; t += step) {
        float sum = 0.0f;
        if (m0 + t < a.M) {
            const float* col = a.row_ssq + m0 + t;
#pragma unroll 8
            for (int p = 0; p < a.ssq_parts; ++p) sum += col[(size_t)p * a.M];
        }
        out[t] = rsqrtf(sum / (float)a.ssq_width + a.ssq_eps);
    }
}

// ---- PTX wrappers --------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait; false = gave up (abort flag set)
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// (bounded both by a number of tries and by wall time: a try may itself block for a while)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t max_spin = MAX_SPIN,
                                          unsigned long long max_wait_ns = MAX_WAIT_NS) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it < max_spin; ++it) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if ((it & 1023u) == 1023u) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > max_wait_ns) break;
        }
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32"
        " {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte
// swizzle: 8-row groups 1024 bytes apart (SBO), version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                                // leading byte offset (unused here)
    d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset
    d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                                // SWIZZLE_128B
    return d;
}

// Instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = NT.
__host__ __device__ constexpr uint32_t umma_idesc(int nt) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(nt >> 3) << 17) |
           ((uint32_t)(TILE_N >> 4) << 24);
}

// One chunk of the epilogue: this thread's 16 consecutive tokens (tok0 ..) of output row n.
// `scale` (may be null): 1 / rms of these 16 tokens, applied to the accumulators first.
__device__ __forceinline__ void store_chunk(const GemmArgs& a, const uint32_t* r_in, int n, bool n_ok,
                                            float bias, int tok0, int lane, int split,
                                            const float* scale = nullptr) {
    uint32_t r[16];
#pragma unroll
    for (int j = 0; j < 16; ++j)
        r[j] = scale ? __float_as_uint(__uint_as_float(r_in[j]) * scale[j]) : r_in[j];
    if (a.epi == EPI_SWIGLU) {
        // Lanes come in pairs: the even lane holds the gate row, the odd lane the up row of the
        // same output column, both for these 16 tokens.  They swap halves (one shuffle per two
        // tokens), then the even lane finishes the even tokens and the odd lane the odd ones, so
        // every lane does half of the work instead of every other lane doing all of it.
        const bool even = (lane & 1) == 0;
        __nv_bfloat16* o = (__nv_bfloat16*)a.out + (size_t)(tok0 + (even ? 0 : 1)) * a.ldo + (n >> 1);
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
            const float keep = __uint_as_float(even ? r[2 * jj] : r[2 * jj + 1]);
            const float send = __uint_as_float(even ? r[2 * jj + 1] : r[2 * jj]);
            const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
            const float g = even ? keep : recv, u = even ? recv : keep;
            const int tok = tok0 + 2 * jj + (even ? 0 : 1);
            if (tok < a.M && n_ok)
                o[(size_t)(2 * jj) * a.ldo] = __float2bfloat16_rn(__fdividef(g * u, 1.0f + __expf(-g)));
        }
    } else if (a.epi == EPI_ACCUM && a.bias == nullptr) {
        // out += acc as a reduction at the memory side: nothing comes back, so a chunk does not
        // wait a round trip for the old values (each element gets exactly one add: same bits)
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + j;
            if (tok < a.M && n_ok)
                asm volatile("red.global.add.f32 [%0], %1;"
                             ::"l"((float*)a.out + (size_t)tok * a.ldo + n), "f"(__uint_as_float(r[j]))
                             : "memory");
        }
    } else if (a.epi == EPI_ACCUM) {
        // all loads of the chunk first, so that they are in flight together
        float old[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + j;
            old[j] = (tok < a.M && n_ok) ? ((const float*)a.out)[(size_t)tok * a.ldo + n] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + j;
            if (tok < a.M && n_ok)
                ((float*)a.out)[(size_t)tok * a.ldo + n] = old[j] + __uint_as_float(r[j]) + bias;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + j;
            const float v = __uint_as_float(r[j]) + bias;
            if (tok < a.M && n_ok) {
                if (a.epi == EPI_PARTIAL)
                    a.partial[((size_t)split * a.M + tok) * a.N + n] = v;
                else if (a.out_dtype == MF_DTYPE_F32)
                    ((float*)a.out)[(size_t)tok * a.ldo + n] = v;
                else
                    ((__nv_bfloat16*)a.out)[(size_t)tok * a.ldo + n] = __float2bfloat16_rn(v);
            }
        }
    }
}

template <int NT> struct TmemCols { static constexpr int value = NT < 32 ? 32 : NT; };

template <int NT, int STAGES>
__global__ void __launch_bounds__(128)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const GemmArgs a) {
    constexpr int B_BYTES = NT * TILE_K * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int TMEM_COLS = TmemCols<NT>::value;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);   // full[S], empty[S], acc
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* scale_s = (float*)(tmem_slot + 2);        // [NT] 1 / rms of this tile's tokens

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * NT;                  // first token of this tile
    const int n0 = blockIdx.y * TILE_N;              // first row of W
    const int split = blockIdx.z;
    const int kblocks = (a.K + TILE_K - 1) / TILE_K;
    const int kb0 = split * a.kblocks_per_split;
    const int kb1 = min(kblocks, kb0 + a.kblocks_per_split);
    const int n_iter = kb1 - kb0;

    if (tid == 0) {
        // the token operand's descriptor is first used after the wait below: fetch it now
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[STAGES + s]), 1);
        }
        mbar_init(smem_u32(&bars[2 * STAGES]), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ------------------------------------------------------------
        // The weights are constant over the step: their first tiles are requested before the
        // kernel waits for the one before it, so that they stream in while that one finishes.
        const int pre = n_iter < STAGES ? n_iter : STAGES;
        for (int i = 0; i < pre; ++i) {
            const uint32_t full = smem_u32(&bars[i]);
            mbar_expect_tx(full, STAGE_BYTES);
            tma_load_2d(smem_u32(smem + i * STAGE_BYTES), &map_w, (kb0 + i) * TILE_K, n0, full);
        }
        // a CTA with only a few tiles beyond its ring asks for them in L2, so that the refill
        // after the first MMAs is not a trip to HBM on the step's critical path
        if (n_iter <= STAGES + 2)
            for (int i = pre; i < n_iter; ++i)
                asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                             ::"l"(&map_w), "r"((kb0 + i) * TILE_K), "r"(n0) : "memory");
        pdl_wait();
        for (int i = 0; i < pre; ++i)
            tma_load_2d(smem_u32(smem + i * STAGE_BYTES) + A_BYTES, &map_x, (kb0 + i) * TILE_K, m0,
                        smem_u32(&bars[i]));
        for (int i = pre; i < n_iter; ++i) {
            const int s = i % STAGES;
            const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
            if (!mbar_wait(smem_u32(&bars[STAGES + s]), ph ^ 1u, abort_flag)) break;
            const uint32_t full = smem_u32(&bars[s]);
            mbar_expect_tx(full, STAGE_BYTES);
            const uint32_t dst = smem_u32(smem + s * STAGE_BYTES);
            tma_load_2d(dst, &map_w, (kb0 + i) * TILE_K, n0, full);
            tma_load_2d(dst + A_BYTES, &map_x, (kb0 + i) * TILE_K, m0, full);
        }
    } else {
        pdl_wait();          // every other thread: nothing below may run ahead of the kernel before
    }
    // the tokens' 1 / rms, by the two warps that have nothing to do while the weights stream
    if (a.row_ssq != nullptr && warp >= 2) row_scales(a, m0, NT, scale_s, tid - 64, 64);
    if (warp == 1 && lane == 0) {
        // ---- MMA issuer --------------------------------------------------------------
        constexpr uint32_t idesc = umma_idesc(NT);
        bool ok = true;
        for (int i = 0; i < n_iter && ok; ++i) {
            const int s = i % STAGES;
            const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
            ok = mbar_wait(smem_u32(&bars[s]), ph, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
            const uint64_t da = umma_desc(sa), db = umma_desc(sa + A_BYTES);
#pragma unroll
            for (int k = 0; k < TILE_K / 16; ++k) {
                // 16 k = 32 bytes further along the swizzled row: +2 in 16-byte units
                tc_mma(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                       (i > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit(smem_u32(&bars[STAGES + s]));      // frees the stage when the MMAs are done
        }
        if (ok) tc_commit(smem_u32(&bars[2 * STAGES]));  // accumulator complete
    }
    __syncwarp();

    // ---- epilogue: all four warps, warp w owns TMEM lanes 32w..32w+31 -------------------
    if (a.row_ssq != nullptr) __syncthreads();           // the scales are in shared memory
    const bool acc_ok = mbar_wait(smem_u32(&bars[2 * STAGES]), 0u, abort_flag);
    tc_fence_after();
    if (acc_ok) {
        const int n = n0 + warp * 32 + lane;
        const bool n_ok = n < a.N;
        const float bias = (a.bias != nullptr && n_ok && a.epi != EPI_PARTIAL) ? a.bias[n] : 0.0f;
#pragma unroll 1
        for (int c0 = 0; c0 < NT; c0 += 16) {
            if (m0 + c0 >= a.M) break;                   // uniform across the CTA
            uint32_t r[16];
            tc_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
            tc_wait_ld();
            store_chunk(a, r, n, n_ok, bias, m0 + c0, lane, split,
                        a.row_ssq != nullptr ? scale_s + c0 : nullptr);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0) {
            atomicOr(a.status, MF_STATUS_WAIT_TIMEOUT);
            // give copies that are still in flight time to land before the memory is reused
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------
// Few tokens, the product that completes the residual stream (out += x W^T): split along K
// over a CLUSTER of CSPLIT CTAs (grid z = cluster z), whose partial tiles never leave the
// chip.  Main loop as in gemm_tc_kernel.  Then, by distributed shared memory:
//   1. as soon as its accumulator is complete, CTA r sends its partial sums of token t (all
//      128 columns of the tile) to the CTA that owns the token (rank t mod CSPLIT), into a
//      buffer of that CTA's shared memory that nothing else uses; meanwhile it fetches the old
//      residual values of its own tokens, the bias and the norm's weights: then one cluster
//      barrier
//   2. every CTA adds the CSPLIT partial sums of its tokens in rank order (reproducible), adds
//      them (and the bias) into `out`, and, if asked, writes the next norm's x' = h * g and each
//      token's sum of h^2 over the tile's 128 columns (see the head of this file).
// No partial sums in global memory, no kernel to add them, and the norm that follows is left
// with a scale that the next product applies.
// ------------------------------------------------------------------------------------------
#define CSPLIT 8

__device__ __forceinline__ uint32_t rank_in_cluster() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float a) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int NT, int STAGES>
__global__ void __launch_bounds__(128)
gemm_tc_cluster_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                       const GemmArgs a) {
    constexpr int B_BYTES = NT * TILE_K * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int TMEM_COLS = TmemCols<NT>::value;
    constexpr int TPO = NT / CSPLIT;                             // tokens a CTA owns: rank, rank + CSPLIT, ..
    constexpr int PART_BYTES = CSPLIT * TILE_N * TPO * 4;        // the partial sums sent to this CTA
    static_assert(TPO >= 2 && TPO % 2 == 0, "a token tile of at least 16 tokens");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* part = (float*)(smem + STAGES * STAGE_BYTES);         // [src rank][owned token][column]
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES + PART_BYTES);   // full[S], empty[S], acc
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* scale_s = (float*)(tmem_slot + 2);        // [NT] 1 / rms of this tile's tokens

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * NT;
    const int n0 = blockIdx.y * TILE_N;
    const uint32_t rank = rank_in_cluster();         // = blockIdx.z: the K split
    const int kblocks = (a.K + TILE_K - 1) / TILE_K;
    const int kb0 = (int)rank * a.kblocks_per_split;
    const int kb1 = min(kblocks, kb0 + a.kblocks_per_split);
    const int n_iter = max(0, kb1 - kb0);

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[STAGES + s]), 1);
        }
        mbar_init(smem_u32(&bars[2 * STAGES]), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer (weights first: they are constant over the step) --------------------
        const int pre = n_iter < STAGES ? n_iter : STAGES;
        for (int i = 0; i < pre; ++i) {
            const uint32_t full = smem_u32(&bars[i]);
            mbar_expect_tx(full, STAGE_BYTES);
            tma_load_2d(smem_u32(smem + i * STAGE_BYTES), &map_w, (kb0 + i) * TILE_K, n0, full);
        }
        if (n_iter <= STAGES + 2)
            for (int i = pre; i < n_iter; ++i)
                asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                             ::"l"(&map_w), "r"((kb0 + i) * TILE_K), "r"(n0) : "memory");
        pdl_wait();
        for (int i = 0; i < pre; ++i)
            tma_load_2d(smem_u32(smem + i * STAGE_BYTES) + A_BYTES, &map_x, (kb0 + i) * TILE_K, m0,
                        smem_u32(&bars[i]));
        for (int i = pre; i < n_iter; ++i) {
            const int s = i % STAGES;
            const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
            if (!mbar_wait(smem_u32(&bars[STAGES + s]), ph ^ 1u, abort_flag)) break;
            const uint32_t full = smem_u32(&bars[s]);
            mbar_expect_tx(full, STAGE_BYTES);
            const uint32_t dst = smem_u32(smem + s * STAGE_BYTES);
            tma_load_2d(dst, &map_w, (kb0 + i) * TILE_K, n0, full);
            tma_load_2d(dst + A_BYTES, &map_x, (kb0 + i) * TILE_K, m0, full);
        }
    } else {
        pdl_wait();
    }
    if (a.row_ssq != nullptr && warp >= 2) row_scales(a, m0, NT, scale_s, tid - 64, 64);
    if (warp == 1 && lane == 0) {
        // ---- MMA issuer ---------------------------------------------------------------------
        constexpr uint32_t idesc = umma_idesc(NT);
        bool ok = true;
        for (int i = 0; i < n_iter && ok; ++i) {
            const int s = i % STAGES;
            const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
            ok = mbar_wait(smem_u32(&bars[s]), ph, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
            const uint64_t da = umma_desc(sa), db = umma_desc(sa + A_BYTES);
#pragma unroll
            for (int k = 0; k < TILE_K / 16; ++k)
                tc_mma(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                       (i > 0 || k > 0) ? 1u : 0u);
            tc_commit(smem_u32(&bars[STAGES + s]));
        }
        if (ok && n_iter > 0) tc_commit(smem_u32(&bars[2 * STAGES]));
    }
    __syncwarp();

    // what this CTA's own tokens need besides the sums: asked for now, used after the barrier.
    // A thread is a column of the tile in both halves of the epilogue.
    const int n_local = warp * 32 + lane;
    const int n = n0 + n_local;
    const bool n_ok = n < a.N;
    const float bias = (a.bias != nullptr && n_ok) ? a.bias[n] : 0.0f;
    const float g = (a.prep_x != nullptr && n_ok) ? a.prep_g[n] : 0.0f;
    float old[TPO];
#pragma unroll
    for (int i = 0; i < TPO; ++i) {
        const int tok = m0 + (int)rank + i * CSPLIT;
        old[i] = (a.epi == EPI_ACCUM && tok < a.M && n_ok) ? ((const float*)a.out)[(size_t)tok * a.ldo + n] : 0.0f;
    }

    // ---- 1. the accumulator is complete: token t's partial sums go to CTA t mod CSPLIT -------------
    const bool acc_ok = n_iter > 0 ? mbar_wait(smem_u32(&bars[2 * STAGES]), 0u, abort_flag) : true;
    tc_fence_after();
    {
        // in the owner: part[(src rank * TPO + t / CSPLIT) * 128 + column]: the 32 lanes of a warp
        // write 128 consecutive bytes
        const uint32_t mine = smem_u32(part + (size_t)rank * TPO * TILE_N + n_local);
#pragma unroll 1
        for (int c0 = 0; c0 < NT; c0 += 16) {
            if (m0 + c0 >= a.M) break;
            uint32_t r[16];
            if (acc_ok && n_iter > 0) {
                tc_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
                tc_wait_ld();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
            // tokens c0 + o and c0 + o + 8 belong to owner o, as its tokens c0 / 8 and c0 / 8 + 1
#pragma unroll
            for (int o = 0; o < CSPLIT; ++o) {
                const uint32_t dst = map_to_rank(mine, (uint32_t)o) + (uint32_t)((c0 / CSPLIT) * TILE_N * 4);
                st_cluster_f32(dst, __uint_as_float(r[o]));
                st_cluster_f32(dst + TILE_N * 4, __uint_as_float(r[o + 8]));
            }
        }
    }
    // Every thread of every CTA of the cluster comes here, whatever happened above (a wait that
    // ran out only sets the abort flag): the cluster's barrier cannot be left waiting.  It also
    // orders the scales in this CTA's shared memory before their use below.
    cluster_barrier();

    // ---- 2. this CTA's tokens: sums in rank order, residual, the next norm's input -----------------
    float* sq_s = scale_s + NT;                       // [4 warps][TPO]
#pragma unroll
    for (int i = 0; i < TPO; ++i) {
        const int t = (int)rank + i * CSPLIT;
        const int tok = m0 + t;
        float sq = 0.0f;
        if (tok < a.M && n_ok) {
            float v = 0.0f;
#pragma unroll
            for (int s = 0; s < CSPLIT; ++s) v += part[((size_t)s * TPO + i) * TILE_N + n_local];
            if (a.row_ssq != nullptr) v *= scale_s[t];
            const float hn = old[i] + v + bias;
            ((float*)a.out)[(size_t)tok * a.ldo + n] = hn;
            if (a.prep_x != nullptr) {
                a.prep_x[(size_t)tok * a.ldp + n] = __float2bfloat16_rn(hn * g);
                sq = hn * hn;
            }
        }
        if (a.prep_x != nullptr) {
            sq = warp_sum(sq);
            if (lane == 0) sq_s[warp * TPO + i] = sq;
        }
    }
    if (a.prep_x != nullptr) {
        __syncthreads();
        if (tid < TPO && m0 + (int)rank + tid * CSPLIT < a.M)
            a.prep_ssq[(size_t)blockIdx.y * a.M + m0 + (int)rank + tid * CSPLIT] =
                (sq_s[tid] + sq_s[TPO + tid]) + (sq_s[2 * TPO + tid] + sq_s[3 * TPO + tid]);
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0) {
            atomicOr(a.status, MF_STATUS_WAIT_TIMEOUT);
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// What a wait that runs out does, shown without a product around it: one thread waits, with
// the limits it is given, on a barrier that nothing ever arrives at (no copy in flight, no
// tensor memory held).  The wait gives up, the kernel sets MF_STATUS_WAIT_TIMEOUT in the
// status word as the product kernels do, and returns; the context stays usable.
__global__ void wait_probe_kernel(unsigned* status, uint32_t max_spin, unsigned long long max_wait_ns,
                                  unsigned long long* waited_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const unsigned long long t0 = global_ns();
        const bool ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag, max_spin, max_wait_ns);
        if (waited_ns) *waited_ns = global_ns() - t0;
        if (!ok) atomicOr(status, MF_STATUS_WAIT_TIMEOUT);
    }
}

extern "C" int mf_wait_probe(unsigned* status, unsigned max_spin, unsigned long long max_wait_ns,
                             unsigned long long* waited_ns, cudaStream_t stream) {
    if (status == nullptr) return MF_ERR_ARGUMENT;
    // the probe may never wait longer than a product kernel would
    if (max_spin > MAX_SPIN) max_spin = MAX_SPIN;
    if (max_wait_ns > MAX_WAIT_NS) max_wait_ns = MAX_WAIT_NS;
    wait_probe_kernel<<<1, 32, 0, stream>>>(status, max_spin, max_wait_ns, waited_ns);
    return MF_LAUNCH_CHECK();
}

// adds the K splits in order: out (+)= sum_s partial[s] + bias
template <typename TO>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, const float* __restrict__ bias,
                                     TO* __restrict__ out, long long ldo, int M, int N, int splits,
                                     int accumulate) {
    pdl_prologue();
    const long long total = (long long)M * N;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(idx % N);
        const long long m = idx / N;
        float v = 0.0f;
        for (int s = 0; s < splits; ++s) v += partial[(size_t)s * total + idx];
        if (bias) v += bias[n];
        TO* o = out + m * ldo + n;
        if (accumulate) v += to_f32(*o);
        *o = from_f32<TO>(v);
    }
}

// ---- host side -------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// bf16 matrix [rows][K] with `ld` elements between rows; box = [box_rows][64]
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return MF_ERR_NO_TENSORMAP;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TILE_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : MF_ERR_TENSORMAP;
}

struct MapKey {
    const void* ptr; int rows, K, box; long long ld;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && K == o.K && box == o.box && ld == o.ld;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ (size_t)k.rows * 1315423911u ^ (size_t)k.K * 2654435761u ^
               (size_t)k.box * 97u ^ (size_t)k.ld * 31u;
    }
};

// tensor maps of weights are made once and kept (weights do not move)
static int weight_map(CUtensorMap* out, const void* ptr, int rows, int K, long long ld) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    MapKey key{ptr, rows, K, TILE_N, ld};
    auto it = cache.find(key);
    if (it == cache.end()) {
        CUtensorMap m;
        if (int e = make_map(&m, ptr, rows, K, ld, TILE_N)) return e;
        it = cache.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}

template <int NT, int STAGES>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a, int splits,
                  cudaStream_t stream) {
    constexpr int smem = STAGES * (A_BYTES + NT * TILE_K * 2) + 1024 + 256 + NT * 4;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<NT, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((a.M + NT - 1) / NT, (a.N + TILE_N - 1) / TILE_N, splits);
    mf_launch(gemm_tc_kernel<NT, STAGES>, dim3(grid), dim3(128), smem, stream, mw, mx, a);
    return MF_LAUNCH_CHECK();
}


template <int NT, int STAGES>
static int launch_cluster(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a,
                          cudaStream_t stream) {
    constexpr int smem = STAGES * (A_BYTES + NT * TILE_K * 2) + TILE_N * NT * 4 + 1024 + 256 + NT * 4 + NT * 2;
    static bool configured[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MF_ERR_UNSUPPORTED;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_cluster_kernel<NT, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.M + NT - 1) / NT, (a.N + TILE_N - 1) / TILE_N, CSPLIT);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = 1;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = CSPLIT;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = mf_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, gemm_tc_cluster_kernel<NT, STAGES>, mw, mx, a);
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// Many tokens: a PAIR of CTAs (a cluster of two SMs) works on one 256 x NT tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 weight rows and its own half of the
// NT tokens, so an SM moves half the operand bytes per MMA clock of the one-CTA kernel; that
// leaves room for a TMA ring that covers an L2 round trip.  The kernel is persistent (one pair
// per two SMs walks over the tiles) and keeps two accumulators in tensor memory, so the four
// epilogue warps of a tile run while the MMA thread is already on the next tile.
//
//   warp 0, one thread   TMA producer (both CTAs); both CTAs' copies complete on the
//                        LEADER's (rank 0) "full" barrier, which the leader arms for both
//   warp 1, one thread   MMA issuer, leader CTA only; tcgen05.commit multicasts to both CTAs'
//                        "empty" barriers (stage free) and "accumulator full" barriers
//   warps 2-9            epilogue of the CTA's own 128 accumulator rows: two groups of four warps
//                        (a warp reads the 32 tensor-memory lanes of its index mod 4) that take
//                        alternate 16-token chunks, each loading its next chunk from tensor memory
//                        while it stores the one before; when done they arrive on the leader's
//                        "accumulator empty" barrier (remote for rank 1)
// No load is multicast: each CTA fetches its own tiles.
//
// DUAL: a pair takes two neighbouring token tiles of one weight tile at once.  A stage then
// holds the 128 weight rows once and both token halves, every k-block feeds both accumulators,
// and the operand bytes a pair pulls per flop fall by a quarter (256 + 2 NT rows instead of
// 2 (256 + NT)).  The two accumulators are then both in use, so a tile's epilogue no longer
// hides behind the next tile's main loop: the form is for products whose tiles make one or two
// rounds over the pairs.  An element's sum is the same in either form (k ascending, one
// accumulator).
// ------------------------------------------------------------------------------------------
#define PAIR_THREADS 320
#define PAIR_EPI_WARPS 8
#define PEER_BIT_MASK 0xFEFFFFFFu      // clears the CTA-rank bit of a shared::cluster address

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(leader_bar)
        : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {   // arrives in both CTAs
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
        " [%0], %1;"
        ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t cta_rank) {
    asm volatile(
        "{\n .reg .b32 ra;\n mapa.shared::cluster.u32 ra, %0, %1;\n"
        " mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n}\n"
        ::"r"(bar), "r"(cta_rank) : "memory");
}

// The order in which the pairs walk the tiles.  Tiles that run side by side fetch what they share
// once (they stream along K in step, so L2 serves the others); what a later round needs again
// comes from memory again.  With few token tiles all of them run beside each other for a weight
// tile.  With many (8,192 tokens and more) that order would fetch every token row once per weight
// tile, gigabytes for a down projection; the token tiles are therefore taken in groups of
// `group_m`, and within a group the weight tiles change slowest, so that a round of tiles is a
// block of about as many weight tiles as token tiles.
__device__ __forceinline__ void pair_tile_at(int tile, int tiles_m, int tiles_n, int group_m,
                                             int& mi, int& ni) {
    const int per_group = group_m * tiles_n;
    const int g = tile / per_group, r = tile - g * per_group;
    const int width = min(group_m, tiles_m - g * group_m);     // the last group may be narrower
    ni = r / width;
    mi = g * group_m + (r - ni * width);
}

template <int NT, int STAGES, bool DUAL>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const GemmArgs a, int tiles_m, int tiles_n, int group_m, int total_tiles) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int HALF_B = (NT / 2) * TILE_K * 2;            // this CTA's half of one token tile
    constexpr int B_BYTES = (DUAL ? 2 : 1) * HALF_B;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int M_STEP = (DUAL ? 2 : 1) * NT;              // tokens a pair takes per tile of its walk
    constexpr int TMEM_COLS = 2 * NT <= 256 ? 256 : 512;      // two accumulators of NT columns (a power of two is allocated)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;                    // [STAGES]  leader's are used
    uint64_t* empty = bars + STAGES;          // [STAGES]  each CTA waits on its own
    uint64_t* acc_full = bars + 2 * STAGES;   // [2]       each CTA waits on its own
    uint64_t* acc_empty = acc_full + 2;       // [2]       leader's are used
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int kblocks = (a.K + TILE_K - 1) / TILE_K;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 2 * PAIR_EPI_WARPS);   // the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                       // both CTAs' barriers exist
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ------------------------------------------------------------
        int it = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
            int mi, ni;
            pair_tile_at(tile, tiles_m, tiles_n, group_m, mi, ni);
            const int m0 = mi * M_STEP, n0 = ni * 256;
            const bool two = DUAL && m0 + NT < a.M;           // the second token tile has tokens
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1u, abort_flag)) { ok = false; break; }
                const uint32_t leader_full = smem_u32(&full[s]) & PEER_BIT_MASK;
                if (rank == 0)
                    mbar_expect_tx(smem_u32(&full[s]), 2 * (A_BYTES + (two ? 2 : 1) * HALF_B));
                const uint32_t dst = smem_u32(smem + s * STAGE_BYTES);
                tma_load_2d_pair(dst, &map_w, kb * TILE_K, n0 + (int)rank * TILE_N, leader_full);
                tma_load_2d_pair(dst + A_BYTES, &map_x, kb * TILE_K, m0 + (int)rank * (NT / 2),
                                 leader_full);
                if (two)
                    tma_load_2d_pair(dst + A_BYTES + HALF_B, &map_x, kb * TILE_K,
                                     m0 + NT + (int)rank * (NT / 2), leader_full);
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---- MMA issuer (leader) -------------------------------------------------------
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) |
                                   ((uint32_t)(256 >> 4) << 24);
        int it = 0, tile_i = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, ++tile_i) {
            // DUAL: both accumulators belong to this tile (barrier 0 stands for the two)
            const int b = DUAL ? 0 : tile_i & 1;
            const uint32_t u = (uint32_t)(DUAL ? tile_i : tile_i >> 1);
            int mi, ni;
            pair_tile_at(tile, tiles_m, tiles_n, group_m, mi, ni);
            const bool two = DUAL && mi * M_STEP + NT < a.M;
            ok = mbar_wait(smem_u32(&acc_empty[b]), (u & 1u) ^ 1u, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + (uint32_t)(b * NT);
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                ok = mbar_wait(smem_u32(&full[s]), ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                const uint64_t da = umma_desc(sa), db = umma_desc(sa + A_BYTES);
                const uint64_t db2 = umma_desc(sa + A_BYTES + HALF_B);
#pragma unroll
                for (int k = 0; k < TILE_K / 16; ++k) {
                    tc_mma_pair(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                                (kb > 0 || k > 0) ? 1u : 0u);
                    if (two)
                        tc_mma_pair(tmem_d + (uint32_t)NT, da + (uint64_t)(2 * k),
                                    db2 + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit_pair(smem_u32(&empty[s]));
            }
            if (ok) tc_commit_pair(smem_u32(&acc_full[b]));
        }
    } else if (warp >= 2) {
        // ---- epilogue: this CTA's 128 rows; warp w reads TMEM lanes 32*(w%4) .. ------------
        const int q = warp & 3;
        const int group = (warp - 2) >> 2;            // 0 or 1
        int tile_i = 0;
        for (int tile = pair; tile < total_tiles; tile += n_pairs, ++tile_i) {
            const int b = DUAL ? 0 : tile_i & 1;
            const uint32_t u = (uint32_t)(DUAL ? tile_i : tile_i >> 1);
            int mi, ni;
            pair_tile_at(tile, tiles_m, tiles_n, group_m, mi, ni);
            const int m0 = mi * M_STEP, n0 = ni * 256;
            if (!mbar_wait(smem_u32(&acc_full[b]), u & 1u, abort_flag)) break;
            tc_fence_after();
            const int n = n0 + (int)rank * TILE_N + q * 32 + lane;
            const bool n_ok = n < a.N;
            const float bias = (a.bias != nullptr && n_ok) ? a.bias[n] : 0.0f;
            // DUAL: columns [0, NT) are the first token tile, [NT, 2 NT) the second.  The groups
            // take chunks group, group + 2, ...; a chunk is 16 columns = 16 tokens.
            int n_chunks = (min(a.M - m0, M_STEP) + 15) >> 4;
            n_chunks = n_chunks > group ? (n_chunks - group + 1) >> 1 : 0;      // this group's share
            const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * NT + group * 16);
            uint32_t ra[16], rb[16];
            if (n_chunks > 0) tc_ld16(t0, ra);
#pragma unroll 1
            for (int i = 0; i < n_chunks; i += 2) {
                tc_wait_ld();
                if (i + 1 < n_chunks) tc_ld16(t0 + (uint32_t)((i + 1) * 32), rb);
                store_chunk(a, ra, n, n_ok, bias, m0 + group * 16 + i * 32, lane, 0);
                if (i + 1 < n_chunks) {
                    tc_wait_ld();
                    if (i + 2 < n_chunks) tc_ld16(t0 + (uint32_t)((i + 2) * 32), ra);
                    store_chunk(a, rb, n, n_ok, bias, m0 + group * 16 + (i + 1) * 32, lane, 0);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(smem_u32(&acc_empty[b]), 0);
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0) {
        atomicOr(a.status, MF_STATUS_WAIT_TIMEOUT);
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    cluster_sync_all();              // the partner no longer reads this CTA's memory or barriers
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

static int sm_count();

static int g_pair_group_m = 0;            // > 0: the width of a group of token tiles (tests, measurement)
extern "C" void mf_gemm_pair_group_m(int group_m) { g_pair_group_m = group_m; }

template <int NT, int STAGES, bool DUAL>
static int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a,
                       cudaStream_t stream) {
    constexpr int smem = STAGES * (A_BYTES + (DUAL ? 2 : 1) * (NT / 2) * TILE_K * 2) + 1024 + 256;
    static_assert(smem <= 227 * 1024, "the ring does not fit an SM's shared memory");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<NT, STAGES, DUAL>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int step = (DUAL ? 2 : 1) * NT;
    const int tiles_m = (a.M + step - 1) / step, tiles_n = (a.N + 255) / 256;
    const int total = tiles_m * tiles_n;
    int pairs = sm_count() / 2;
    // groups of token tiles such that a round of tiles is about square (as many weight tiles
    // as token tiles, 9 x 9 for 74 pairs), all groups equally wide
    int side = 1;
    while ((side + 1) * (side + 1) <= pairs) ++side;
    const int across = tiles_n < side ? tiles_n : side;
    const int want_m = (pairs + across - 1) / across;
    const int groups = (tiles_m + want_m - 1) / want_m;
    int group_m = (tiles_m + groups - 1) / groups;
    if (g_pair_group_m > 0) group_m = g_pair_group_m < tiles_m ? g_pair_group_m : tiles_m;
    if (pairs > total) pairs = total;
    mf_launch(gemm_pair_kernel<NT, STAGES, DUAL>, dim3(2 * pairs), dim3(PAIR_THREADS), smem, stream, mw, mx,
              a, tiles_m, tiles_n, group_m, total);
    return MF_LAUNCH_CHECK();
}

static int sm_count() { return mf_sm_count(); }

// How the CTA-pair kernel cuts a product: the token tile and whether a pair takes two token
// tiles at once (DUAL).  A model of the kernel's time picks them; its figures are measured on
// this kernel (2,048 to 8,192 tokens, K 1,792 to 18,944):
//   * operand bytes: every k-block a pair pulls 256 weight rows and its tokens' rows, 128 bytes
//     each, through L2, and all pairs together get 11.8 TB/s (a 208-token tile takes 0.905 of a
//     256-token one: the ratio of the bytes, not of the flops);
//   * tensor cores: 23.4 TFLOP/s a pair with every pair at work (the clock under load);
//   * rounds: the pairs walk the tiles in step, so the last round counts in full
//     (14 weight tiles x 8 token tiles of 256 are 112 tiles for 74 pairs; 10 token tiles of 208
//     are 140 tiles and two full rounds);
//   * what is not hidden: the last tile's epilogue, and with DUAL every tile's (both
//     accumulators are in use, so none is free for the next tile's main loop).
// DUAL therefore wins where the tiles make one or two rounds, the more the longer K is (the
// down projection of a 2,048-token prompt: 181 against 217 us; the O projection: 44 against 50);
// it is not considered beyond two rounds.  An element's sum does not depend
// on the cut (k ascending, one accumulator), so the choice changes no bits.
struct PairPlan { int nt; int dual; };
static int g_pair_dual = -1;              // 0 never, 1 where the model says so, 2 always
// MINFER_B200_PAIR_DUAL or this call (tests compare the two forms bit for bit) sets the mode.
extern "C" void mf_gemm_pair_dual_mode(int mode) { g_pair_dual = mode; }
static PairPlan pair_plan(int M, int N, int K) {
    static const int candidates[] = {256, 224, 208, 192, 160};
    if (g_pair_dual < 0) { const char* ev = getenv("MINFER_B200_PAIR_DUAL"); g_pair_dual = ev ? atoi(ev) : 1; }
    const int allow_dual = g_pair_dual;
    const double pairs = sm_count() / 2, tiles_n = (N + 255) / 256, kb = (K + TILE_K - 1) / TILE_K;
    const double l2_bytes_per_ns = 11800.0 * (pairs / 74.0), pair_flops_per_ns = 23400.0;
    PairPlan best = {256, 0};
    double best_cost = -1.0;
    for (int dual = allow_dual == 2 ? 1 : 0; dual <= (allow_dual ? 1 : 0); ++dual)
        for (int nt : candidates) {
            const int step = (dual ? 2 : 1) * nt;
            const double tiles = (double)((M + step - 1) / step) * tiles_n;
            const double rounds = (double)(long long)((tiles + pairs - 1) / pairs);
            const double bytes = 128.0 * (256 + step), flops = 2.0 * 256 * step * TILE_K;
            const double l2 = tiles * kb * bytes / l2_bytes_per_ns;
            const double tc = rounds * kb * flops / pair_flops_per_ns;
            const double epilogue = (dual ? rounds * 11600.0 : 4000.0) * nt / 256.0;
            double cost = (l2 > tc ? l2 : tc) + epilogue;
            if (dual && rounds > 2 && allow_dual != 2) continue;   // measured for one and two rounds only
            if (best_cost < 0 || cost < best_cost) { best = {nt, dual}; best_cost = cost; }
        }
    return best;
}

// The cut of the CTA-pair kernel for these sizes (it runs products of 256 tokens and more).
extern "C" int mf_gemm_pair_plan(int M, int N, int K, int* token_tile, int* dual) {
    const PairPlan pp = pair_plan(M, N, K);
    *token_tile = pp.nt;
    *dual = pp.dual;
    return 0;
}

// How a product of these sizes is cut: the token tile and the number of K splits.  A
// function of the sizes only (never of the data), so results are reproducible.
extern "C" int mf_gemm_tc_plan(int M, int N, int K, int epi, int* token_tile, int* splits) {
    // many tokens: 128-token tiles with three stages, so that two CTAs share an SM and one's
    // epilogue overlaps the other's main loop (measured faster than 256-token tiles with one
    // CTA per SM for K = 3584: 958 against 847 TFLOP/s)
    int nt = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    const int tiles = ((M + nt - 1) / nt) * ((N + TILE_N - 1) / TILE_N);
    const int kblocks = (K + TILE_K - 1) / TILE_K;
    int s = 1;
    const long long weight_bytes = (long long)N * K * 2;
    if (epi != EPI_SWIGLU && nt <= 64 && weight_bytes <= (16ll << 20)) {
        // small weights (up to 16 MB): their bytes cost next to nothing, the chain of loads of
        // one CTA does (it has STAGES tiles in flight and waits a round trip for each refill).
        // So K is cut until a CTA has 2 k-blocks and asks for all of its weight tiles at once,
        // before it even waits for the kernel before it.  Measured on the Qwen2.5-0.5B shape
        // (64 sequences, 24 layers): 1.50 -> 1.35 ms a step; 4 k-blocks a CTA 1.37-1.39,
        // at most 8 splits 1.39-1.47; a ring twice as deep for grids of at most one CTA an
        // SM gained nothing without the cut and lost 0.08 ms with it.
        s = 2 * sm_count() / tiles;
        if (s > kblocks / 2) s = kblocks / 2;
        if (s > 16) s = 16;
        if (s < 1) s = 1;
    } else if (epi != EPI_SWIGLU && tiles < 200 && kblocks >= 8) {
        // up to two CTAs per SM (the small-token kernels are sized for that), each with at
        // least 4 k-blocks; the partial sums (written and read once) stay under half of the
        // weight bytes: splits * M * N * 8 <= N * K  =>  splits <= K / (8 M)
        const int slots = nt <= 64 ? 2 * sm_count() : sm_count();
        s = slots / tiles;
        if (s > kblocks / 4) s = kblocks / 4;
        if (s > K / (8 * M)) s = K / (8 * M);
        if (s > 16) s = 16;
        if (s < 1) s = 1;
    }
    *token_tile = nt;
    *splits = s;
    return 0;
}

extern "C" long long mf_gemm_tc_workspace_floats(int M, int N, int K, int epi) {
    int nt, s;
    mf_gemm_tc_plan(M, N, K, epi, &nt, &s);
    return s > 1 ? (long long)s * M * N : 0;
}

// What the caller may fold into a product (all null / zero: a plain product).
struct FusedNorm {
    const float* row_ssq;     // consumer: sums of squares [ssq_parts][M] of the norm whose x' this product reads
    int ssq_parts, ssq_width;
    float ssq_eps;
    __nv_bfloat16* prep_x;    // producer (EPI_ACCUM): the next norm's x' [M][N] ...
    long long ldp;
    const float* prep_g;      // ... its weight [N] ...
    float* prep_ssq;          // ... and the sums of squares [parts][M] this product writes
};

static int pair_mode_on() {
    static int pair_mode = -1;            // MINFER_B200_GEMM_PAIR=0 keeps the one-CTA kernel
    if (pair_mode < 0) { const char* ev = getenv("MINFER_B200_GEMM_PAIR"); pair_mode = ev ? atoi(ev) : 1; }
    return pair_mode;
}

// Number of column groups (`parts`) whose sums of squares a residual-completing product of these
// sizes writes, or 0 if no kernel folds the next norm in at these sizes (the caller then adds
// the product in the ordinary way and runs the norm as a kernel).
extern "C" int mf_gemm_tc_prep_parts(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    int nt, splits;
    mf_gemm_tc_plan(M, N, K, EPI_ACCUM, &nt, &splits);
    const int kblocks = (K + TILE_K - 1) / TILE_K;
    // (Folded into the CTA-pair kernel of whole prompts as well it lost: the two norms of a layer
    // cost 19 us at 2,048 tokens, the longer epilogues of the four products 36 us.)
    // Every cluster has to be on the GPU at once, two CTAs to an SM: more column tiles than that
    // allows (hidden 5,120: 40 tiles, 320 CTAs) would run in two rounds, and lost (7.49 -> 7.58 ms
    // a step at the 14B shape); such sizes keep the split with partial sums in memory.
    const int tiles_n = (N + TILE_N - 1) / TILE_N;
    if (nt <= 64 && splits > 1 && kblocks >= CSPLIT && tiles_n * CSPLIT <= 2 * sm_count()) return tiles_n;
    return 0;
}

static int gemm_tc_impl(const void* x, long long ldx, const void* w, long long ldw,
                        const float* bias, void* out, long long ldo, int out_dtype, int M, int N,
                        int K, int epi, float* workspace, int* deferred, unsigned* status,
                        const FusedNorm* f, cudaStream_t stream) {
    if (deferred) *deferred = 0;
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return MF_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return MF_ERR_UNSUPPORTED;
    if (epi == EPI_ACCUM && out_dtype != MF_DTYPE_F32) return MF_ERR_UNSUPPORTED;
    if (epi == EPI_SWIGLU && (out_dtype != MF_DTYPE_BF16 || N % 2 != 0)) return MF_ERR_UNSUPPORTED;
    if (epi < EPI_STORE || epi > EPI_SWIGLU) return MF_ERR_ARGUMENT;
    const bool prep = f != nullptr && f->prep_x != nullptr;
    if (prep && (epi != EPI_ACCUM || f->prep_g == nullptr || f->prep_ssq == nullptr)) return MF_ERR_ARGUMENT;
    if (f != nullptr && f->row_ssq != nullptr && (f->ssq_parts <= 0 || f->ssq_width <= 0)) return MF_ERR_ARGUMENT;
    if (prep && mf_gemm_tc_prep_parts(M, N, K) == 0) return MF_ERR_UNSUPPORTED;
    int nt, splits;
    mf_gemm_tc_plan(M, N, K, epi, &nt, &splits);
    if (splits > 1 && workspace == nullptr && !prep) return MF_ERR_ARGUMENT;
    CUtensorMap mw, mx;
    if (int e = weight_map(&mw, w, N, K, ldw)) return e;
    GemmArgs a = {};
    a.out = out; a.partial = nullptr; a.bias = bias; a.status = status; a.ldo = ldo;
    a.M = M; a.N = N; a.K = K; a.out_dtype = out_dtype; a.kblocks_per_split = 0; a.epi = epi;
    if (f != nullptr) {
        a.row_ssq = f->row_ssq; a.ssq_parts = f->ssq_parts; a.ssq_width = f->ssq_width; a.ssq_eps = f->ssq_eps;
        a.prep_x = f->prep_x; a.ldp = f->ldp; a.prep_g = f->prep_g; a.prep_ssq = f->prep_ssq;
    }
    if (pair_mode_on() && M >= 256 && splits == 1) {
        if (a.row_ssq != nullptr) return MF_ERR_UNSUPPORTED;     // the CTA-pair kernel applies no row scale
        const PairPlan pp = pair_plan(M, N, K);
        const int pnt = pp.nt, dual = pp.dual;
        if (int e = make_map(&mx, x, M, K, ldx, pnt / 2)) return e;
        if (dual)
            switch (pnt) {
                case 224: return launch_pair<224, 5, true>(mw, mx, a, stream);
                case 208: return launch_pair<208, 5, true>(mw, mx, a, stream);
                case 192: return launch_pair<192, 5, true>(mw, mx, a, stream);
                case 160: return launch_pair<160, 6, true>(mw, mx, a, stream);
                default: return launch_pair<256, 4, true>(mw, mx, a, stream);
            }
        switch (pnt) {
            case 224: return launch_pair<224, 6, false>(mw, mx, a, stream);
            case 208: return launch_pair<208, 6, false>(mw, mx, a, stream);
            case 192: return launch_pair<192, 6, false>(mw, mx, a, stream);
            case 160: return launch_pair<160, 6, false>(mw, mx, a, stream);
            default: return launch_pair<256, 6, false>(mw, mx, a, stream);
        }
    }
    if (int e = make_map(&mx, x, M, K, ldx, nt)) return e;
    const int kblocks = (K + TILE_K - 1) / TILE_K;
    if (prep) {
        // few tokens, the residual completed inside the product: K split over a cluster
        a.kblocks_per_split = (kblocks + CSPLIT - 1) / CSPLIT;
        switch (nt) {
            // (a stage fewer than the kernel without a cluster: the buffer for the partial sums
            // takes its place, two CTAs still share an SM)
            case 16: return launch_cluster<16, 5>(mw, mx, a, stream);
            case 32: return launch_cluster<32, 4>(mw, mx, a, stream);
            default: return launch_cluster<64, 3>(mw, mx, a, stream);
        }
    }
    a.partial = workspace;
    a.kblocks_per_split = (kblocks + splits - 1) / splits;
    splits = (kblocks + a.kblocks_per_split - 1) / a.kblocks_per_split;   // no empty split
    a.epi = splits > 1 ? EPI_PARTIAL : epi;
    int e;
    switch (nt) {
        // few tokens: stages sized so that two CTAs share an SM (one's epilogue and prologue
        // overlap the other's stream of weight tiles)
        case 16: e = launch<16, 6>(mw, mx, a, splits, stream); break;
        case 32: e = launch<32, 5>(mw, mx, a, splits, stream); break;
        case 64: e = launch<64, 4>(mw, mx, a, splits, stream); break;
        default: e = launch<128, 3>(mw, mx, a, splits, stream); break;
    }
    if (e || splits == 1) return e;
    if (deferred) {
        *deferred = splits;
        return 0;
    }
    const long long total = (long long)M * N;
    const int threads = 256;
    const long long cap = (long long)sm_count() * 8;
    const int blocks = (int)((total + threads - 1) / threads < cap ? (total + threads - 1) / threads : cap);
    if (out_dtype == MF_DTYPE_F32)
        mf_launch(splitk_reduce_kernel<float>, dim3(blocks), dim3(threads), 0, stream, 
            workspace, bias, (float*)out, ldo, M, N, splits, epi == EPI_ACCUM);
    else
        mf_launch(splitk_reduce_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, 
            workspace, bias, (__nv_bfloat16*)out, ldo, M, N, splits, 0);
    return MF_LAUNCH_CHECK();
}

// out[M][N] (+)= x[M][K] * w[N][K]^T (+ bias).  x, w bfloat16; for EPI_SWIGLU the rows of w
// alternate gate,up and out is [M][N/2] bfloat16.  `workspace` must hold
// mf_gemm_tc_workspace_floats floats when that is not zero.
// `deferred` (may be null): if the product is split along K, the partial sums are LEFT in
// `workspace` as [splits][M][N], nothing is written to `out`, and *deferred receives the number
// of splits, so that the caller's next kernel can add them (and the bias) itself; otherwise
// *deferred is 0 and `out` is complete.
extern "C" int mf_gemm_tc(const void* x, long long ldx, const void* w, long long ldw,
                          const float* bias, void* out, long long ldo, int out_dtype, int M, int N,
                          int K, int epi, float* workspace, int* deferred, unsigned* status,
                          cudaStream_t stream) {
    return gemm_tc_impl(x, ldx, w, ldw, bias, out, ldo, out_dtype, M, N, K, epi, workspace, deferred,
                        status, nullptr, stream);
}

// The same product with a norm folded in on either side (see the head of this file):
// `row_ssq` [ssq_parts][M] (may be null): x is the x' = h * g of a norm over `ssq_width` columns
// with `ssq_eps`; the accumulators of token t are multiplied by its 1 / rms before anything else.
// `prep_x` (may be null; EPI_ACCUM only; sizes for which mf_gemm_tc_prep_parts is not 0): `out`
// is complete when the call returns (no deferred sums), prep_x [M][N] (ldp between rows) holds
// bfloat16(out * prep_g) and prep_ssq [parts][M] the sums of out^2 per column group.
extern "C" int mf_gemm_tc_fused(const void* x, long long ldx, const void* w, long long ldw,
                                const float* bias, void* out, long long ldo, int out_dtype, int M,
                                int N, int K, int epi, float* workspace, int* deferred,
                                const float* row_ssq, int ssq_parts, int ssq_width, float ssq_eps,
                                void* prep_x, long long ldp, const float* prep_g, float* prep_ssq,
                                unsigned* status, cudaStream_t stream) {
    FusedNorm f;
    f.row_ssq = row_ssq; f.ssq_parts = ssq_parts; f.ssq_width = ssq_width; f.ssq_eps = ssq_eps;
    f.prep_x = (__nv_bfloat16*)prep_x; f.ldp = ldp; f.prep_g = prep_g; f.prep_ssq = prep_ssq;
    return gemm_tc_impl(x, ldx, w, ldw, bias, out, ldo, out_dtype, M, N, K, epi, workspace, deferred,
                        status, &f, stream);
}

// out (+)= bias + sum over the K splits left in `partial` ([splits][M][N]) by a deferred
// product, added in split order.
extern "C" int mf_splitk_reduce(const float* partial, int splits, const float* bias, void* out,
                                long long ldo, int out_dtype, int M, int N, int accumulate,
                                cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (splits < 1 || partial == nullptr) return MF_ERR_ARGUMENT;
    if (accumulate && out_dtype != MF_DTYPE_F32) return MF_ERR_UNSUPPORTED;
    const long long total = (long long)M * N;
    const int threads = 256;
    const long long cap = (long long)sm_count() * 8;
    const int blocks = (int)((total + threads - 1) / threads < cap ? (total + threads - 1) / threads : cap);
    if (out_dtype == MF_DTYPE_F32)
        mf_launch(splitk_reduce_kernel<float>, dim3(blocks), dim3(threads), 0, stream, partial, bias, (float*)out, ldo, M,
                                                                    N, splits, accumulate);
    else if (out_dtype == MF_DTYPE_BF16)
        mf_launch(splitk_reduce_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, 
            partial, bias, (__nv_bfloat16*)out, ldo, M, N, splits, 0);
    else
        return MF_ERR_UNSUPPORTED;
    return MF_LAUNCH_CHECK();
}
