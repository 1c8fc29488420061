// Sampling on the device: penalties -> greedy | (top-k -> top-p -> temperature draw).
//
// The pipeline and every rule are the reference's (src/sampler.rs:272-290):
//   * penalties over the distinct tokens of the recent window, frequency then presence
//     then repeat (positive logits divided, others multiplied)      src/sampler.rs:44-76
//   * temperature below 1e-6 is greedy; the first maximum wins      src/sampler.rs:16-26, 284-286
//   * top-k keeps everything >= the k-th largest value (ties stay)  src/sampler.rs:125-137
//   * top-p works on the softmax of the *unscaled* survivors, sorted by descending
//     probability with ties in index order, and keeps up to and including the first entry
//     whose running sum exceeds p                                   src/sampler.rs:149-196
//   * the draw: logits / temp, softmax, first index in ascending order whose running sum
//     reaches r, the last index as fallback                         src/sampler.rs:224-267
// The reference draws r from Rust's StdRng on the CPU; here r comes from Philox4x32-10
// keyed by the seed with the counter (draw number, stream id), so that a sequence's draws
// do not depend on what else is in the batch.  Sums are kept in double where the
// reference uses f64.
//
// One block of 1024 threads works on one row, whatever the batch, so a row's result never
// depends on its neighbours.  Every pass over the row is coalesced (see sample_kernel).  The recent window and the draw counter live in a small
// fixed-size state per sequence: state[slot] = {n_seen, n_draws, ring[64]}.
#include "common.cuh"

#define SMP_THREADS 1024
#define SMP_RECENT 64
#define SMP_STATE_INTS (2 + SMP_RECENT)
#define SMP_SORT_MAX 1024
#define SMP_LIST_MAX 2048

__device__ __forceinline__ unsigned order_key(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__device__ __forceinline__ unsigned philox_uniform_bits(unsigned long long seed, unsigned c0,
                                                        unsigned c1) {
    unsigned k0 = (unsigned)seed, k1 = (unsigned)(seed >> 32);
    unsigned x0 = c0, x1 = c1, x2 = 0u, x3 = 0u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const unsigned hi0 = __umulhi(0xD2511F53u, x0), lo0 = 0xD2511F53u * x0;
        const unsigned hi1 = __umulhi(0xCD9E8D57u, x2), lo1 = 0xCD9E8D57u * x2;
        const unsigned y0 = hi1 ^ x1 ^ k0, y1 = lo1, y2 = hi0 ^ x3 ^ k1, y3 = lo0;
        x0 = y0; x1 = y1; x2 = y2; x3 = y3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return x0;
}

struct SampleArgs {
    float* logits;            // [rows][ld], changed in place
    long long ld;
    int vocab;
    const int* slots;         // [rows] state slot of each row, or null (no penalties, draw 0)
    int* state;               // [n_slots][SMP_STATE_INTS]
    const int* stream_ids;    // [rows] RNG stream of each row, or null (= row index)
    int* out;                 // [rows]
    float temp, top_p, repeat, frequency, presence;
    int top_k;
    unsigned long long seed;
    int update_state;         // append the sampled token to the window, count the draw
};

// ---- block-wide reductions: shuffles inside a warp, 32 partial results through shared memory ----
__device__ __forceinline__ double warp_sum_double(double v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
// every thread gets the block's sum; `buf` holds 32 doubles
__device__ double block_sum_double(double v, double* buf) {
    v = warp_sum_double(v);
    if ((threadIdx.x & 31) == 0) buf[threadIdx.x >> 5] = v;
    __syncthreads();
    double r = buf[threadIdx.x & 31];
    r = warp_sum_double(r);
    __syncthreads();
    return r;
}
__device__ int block_sum_int(int v, int* buf) {
    v = warp_sum_int(v);
    if ((threadIdx.x & 31) == 0) buf[threadIdx.x >> 5] = v;
    __syncthreads();
    int r = buf[threadIdx.x & 31];
    r = warp_sum_int(r);
    __syncthreads();
    return r;
}
__device__ int block_min_int(int v, int* buf) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, off));
    if ((threadIdx.x & 31) == 0) buf[threadIdx.x >> 5] = v;
    __syncthreads();
    int r = buf[threadIdx.x & 31];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) r = min(r, __shfl_xor_sync(0xffffffffu, r, off));
    __syncthreads();
    return r;
}
// The k-th largest of `n` values in shared memory (1 <= k <= n), by radix selection over the
// order-preserving bits; every thread of the block calls it and gets the value.
__device__ float kth_largest(const float* vals, int n, int k, unsigned* hist, unsigned* sh_prefix,
                             int* sh_left) {
    unsigned prefix = 0u, mask = 0u;
    int k_left = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (threadIdx.x < 256) hist[threadIdx.x] = 0u;
        __syncthreads();
        for (int e = threadIdx.x; e < n; e += SMP_THREADS) {
            const unsigned key = order_key(vals[e]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // the highest bin at which the count from the top reaches k_left: lane l holds the
            // bins 255 - 8 l down to 248 - 8 l
            const int lane = threadIdx.x;
            int mine[8], total = 0;
#pragma unroll
            for (int b = 0; b < 8; ++b) { mine[b] = (int)hist[255 - 8 * lane - b]; total += mine[b]; }
            int incl = total;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += up;
            }
            const unsigned reach = __ballot_sync(0xffffffffu, incl >= k_left);
            const int owner = reach != 0u ? __ffs(reach) - 1 : 31;
            if (lane == owner) {
                int left = k_left - (incl - total);
                int b = 0;
                for (; b < 7; ++b) {
                    if (mine[b] >= left) break;
                    left -= mine[b];
                }
                int bin = 255 - 8 * lane - b;
                if (reach == 0u) { bin = 0; left = 1; }      // fewer than k values: the lowest bin
                *sh_prefix = prefix | ((unsigned)bin << shift);
                *sh_left = left;
            }
        }
        __syncthreads();
        prefix = *sh_prefix;
        k_left = *sh_left;
        mask |= 255u << shift;
        __syncthreads();
    }
    return key_value(prefix);
}

// The row is cut into 32 consecutive ranges, one per warp; a warp walks its range in rows of
// 32 consecutive indices, lane l taking the l-th: loads are coalesced and (warp, row, lane)
// is the index order, which the draw and the ties of top-p need.
__global__ void __launch_bounds__(SMP_THREADS, 1) sample_kernel(SampleArgs a) {
    pdl_prologue();
    __shared__ double dbuf[32];
    __shared__ float fscratch[33];
    __shared__ int ibuf[32];
    __shared__ float sort_p[SMP_SORT_MAX];
    __shared__ int sort_i[SMP_SORT_MAX];
    __shared__ unsigned hist[256];
    __shared__ double hsum[256];
    __shared__ double wsum[32];
    __shared__ double rowtot[SMP_THREADS];       // the draw: sums of the owner range's rows
    __shared__ float list_v[SMP_LIST_MAX];       // top-k: the candidates of the highest digits
    __shared__ int list_i[SMP_LIST_MAX];
    __shared__ float surv_v[SMP_SORT_MAX];       // top-k: the survivors' logits, beside sort_p / sort_i
    __shared__ unsigned sh_prefix;
    __shared__ int sh_int;
    __shared__ double sh_dbl;

    const int row = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int V = a.vocab;
    float* x = a.logits + (size_t)row * a.ld;
    int* st = (a.slots != nullptr && a.state != nullptr)
                  ? a.state + (size_t)a.slots[row] * SMP_STATE_INTS : nullptr;
    const int n_rows = (V + SMP_THREADS - 1) / SMP_THREADS;    // rows of 32 indices per warp
    const int w_begin = warp * n_rows * 32;                    // may lie beyond V for late warps
#define OWN_ROWS(j, i) for (int j = 0, i = w_begin + lane; j < n_rows; ++j, i += 32)

    // ---- penalties over the distinct tokens of the window -------------------------------
    const bool pen = st != nullptr && (fabsf(a.repeat - 1.0f) >= 1e-6f ||
                                       fabsf(a.frequency) >= 1e-6f || fabsf(a.presence) >= 1e-6f);
    if (pen) {
        const int n_win = min(st[0], SMP_RECENT);
        if (tid < n_win) {
            const int tok = st[2 + tid];
            bool first = true;
            int count = 0;
            for (int i = 0; i < n_win; ++i) {
                if (st[2 + i] == tok) {
                    if (i < tid) first = false;
                    ++count;
                }
            }
            if (first && tok >= 0 && tok < V) {
                float nv = x[tok];
                if (fabsf(a.frequency) >= 1e-6f || fabsf(a.presence) >= 1e-6f) {
                    nv -= (float)count * a.frequency;
                    nv -= a.presence;
                }
                if (fabsf(a.repeat - 1.0f) >= 1e-6f && a.repeat >= 1.0f)
                    nv = nv <= 0.0f ? nv * a.repeat : nv / a.repeat;
                x[tok] = nv;
            }
        }
        __syncthreads();
    }

    int chosen = -1;
    if (a.temp < 1e-6f) {
        // ---- greedy: the first maximum wins ---------------------------------------------
        float best = -INFINITY;
        int best_i = V;                                    // V = "none yet"
#pragma unroll 8
        OWN_ROWS(j, i) {
            if (i < V) {
                const float v = x[i];
                if (best_i == V || v > best) { best = v; best_i = i; }
            }
        }
        const float mx = block_max(best_i == V ? -INFINITY : best, fscratch);
        // lowest index among those equal to the maximum (a NaN row falls back to index 0)
        const int first = block_min_int((best_i != V && best == mx) ? best_i : V, ibuf);
        chosen = first < V ? first : 0;
    } else {
        // ---- top-k, the usual case (k up to a few hundred).  Every thread has the maximum of
        // its own elements; the k-th largest of those 1024 maxima is a lower bound of the k-th
        // largest element (k elements reach it), so whatever passes it is a candidate: about k
        // elements whatever the logits' distribution.  Two passes over the row (maxima; gather
        // of the candidates into shared memory), then everything else (the exact threshold,
        // top-p, the draw) on the short list.
        int n_list = -1;                                   // >= 0: survivors are in surv_v / sort_i
        float list_max = -INFINITY;
        if (a.top_k > 0 && a.top_k < V && a.top_k <= SMP_THREADS) {
            float mx_l = -INFINITY;
#pragma unroll 8
            OWN_ROWS(j, i)
                if (i < V) mx_l = fmaxf(mx_l, x[i]);
            list_max = block_max(mx_l, fscratch);
            list_v[tid] = mx_l;
            __syncthreads();
            const float bound = kth_largest(list_v, SMP_THREADS, a.top_k, hist, &sh_prefix, &sh_int);
            if (tid == 0) sh_int = 0;
            __syncthreads();
            if (bound > -INFINITY) {
#pragma unroll 8
                OWN_ROWS(j, i) {
                    const float v = i < V ? x[i] : -INFINITY;
                    const bool in = i < V && v >= bound;
                    const unsigned lanes = __ballot_sync(0xffffffffu, in);
                    if (lanes != 0u) {
                        int base = 0;
                        if (lane == 0) base = atomicAdd(&sh_int, __popc(lanes));
                        base = __shfl_sync(0xffffffffu, base, 0);
                        const int at = base + __popc(lanes & ((1u << lane) - 1u));
                        if (in && at < SMP_LIST_MAX) {
                            list_v[at] = v;
                            list_i[at] = i;
                        }
                    }
                }
            }
            __syncthreads();
            const int n_cand = sh_int;
            __syncthreads();
            if (n_cand >= a.top_k && n_cand <= SMP_LIST_MAX) {
                const float threshold = kth_largest(list_v, n_cand, a.top_k, hist, &sh_prefix, &sh_int);
                if (tid == 0) sh_int = 0;
                __syncthreads();
                for (int e = tid; e < n_cand; e += SMP_THREADS) {
                    const float v = list_v[e];
                    if (v >= threshold) {                  // ties at the edge stay
                        const int at = atomicAdd(&sh_int, 1);
                        if (at < SMP_SORT_MAX) { surv_v[at] = v; sort_i[at] = list_i[e]; }
                    }
                }
                __syncthreads();
                if (sh_int <= SMP_SORT_MAX) n_list = sh_int;
                __syncthreads();
            }
        }
        if (n_list >= 0) {
            // ---- top-p and the draw over the survivors' list --------------------------------
            int n = n_list;
            int sz = 32;
            while (sz < n) sz <<= 1;
            if (a.top_p > 0.0f && a.top_p < 1.0f) {
                double part = 0.0;
                if (tid < n) part = exp((double)(surv_v[tid] - list_max));
                const float sum_f = (float)block_sum_double(part, dbuf);
                if (tid < sz) sort_p[tid] = tid < n ? expf(surv_v[tid] - list_max) / sum_f : -1.0f;
                if (tid >= n && tid < sz) sort_i[tid] = 0x7fffffff;
                __syncthreads();
                // by (probability descending, index ascending); the logits move along
                for (int size = 2; size <= sz; size <<= 1) {
                    for (int stride = size >> 1; stride > 0; stride >>= 1) {
                        if (tid < sz) {
                            const int partner = tid ^ stride;
                            if (partner > tid) {
                                const bool descending_block = (tid & size) == 0;
                                const float pa = sort_p[tid], pb = sort_p[partner];
                                const int ia = sort_i[tid], ib = sort_i[partner];
                                const bool a_first = pa > pb || (pa == pb && ia < ib);
                                if (a_first != descending_block) {
                                    const float va = surv_v[tid], vb = surv_v[partner];
                                    sort_p[tid] = pb; sort_p[partner] = pa;
                                    sort_i[tid] = ib; sort_i[partner] = ia;
                                    surv_v[tid] = vb; surv_v[partner] = va;
                                }
                            }
                        }
                        __syncthreads();
                    }
                }
                if (tid == 0) {
                    float cum = 0.0f;
                    int keep = n;
                    for (int i = 0; i < n; ++i) {
                        cum += sort_p[i];
                        if (cum > a.top_p) { keep = i + 1; break; }
                    }
                    sh_int = keep;
                }
                __syncthreads();
                n = sh_int;
                __syncthreads();
            }
            // the draw walks the indices in ascending order: sort what is left by index
            if (tid >= n && tid < sz) sort_i[tid] = 0x7fffffff;
            __syncthreads();
            for (int size = 2; size <= sz; size <<= 1) {
                for (int stride = size >> 1; stride > 0; stride >>= 1) {
                    if (tid < sz) {
                        const int partner = tid ^ stride;
                        if (partner > tid) {
                            const bool ascending_block = (tid & size) == 0;
                            const int ia = sort_i[tid], ib = sort_i[partner];
                            if ((ia < ib) != ascending_block) {
                                const float va = surv_v[tid], vb = surv_v[partner];
                                sort_i[tid] = ib; sort_i[partner] = ia;
                                surv_v[tid] = vb; surv_v[partner] = va;
                            }
                        }
                    }
                    __syncthreads();
                }
            }
            const float inv_temp = 1.0f / a.temp;
            const float mx = list_max * inv_temp;          // the maximum always survives
            const float e_t = tid < n ? expf(surv_v[tid] * inv_temp - mx) : 0.0f;
            const double total = block_sum_double((double)e_t, dbuf);
            const float inv_sum = (float)(1.0 / total);
            const float pr = e_t * inv_sum;
            // running sum over the survivors, in index order: inside a warp, then over the warps
            double run = (double)pr;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const double up = __shfl_up_sync(0xffffffffu, run, off);
                if (lane >= off) run += up;
            }
            if (lane == 31) wsum[warp] = run;
            __syncthreads();
            double before = 0.0;
            for (int w = 0; w < warp; ++w) before += wsum[w];
            const double cum = before + run;
            const unsigned draw = st ? (unsigned)st[1] : 0u;
            const unsigned stream = a.stream_ids ? (unsigned)a.stream_ids[row] : (unsigned)row;
            const float r = (float)(philox_uniform_bits(a.seed, draw, stream) >> 8) *
                            (1.0f / 16777216.0f);
            const int first = block_min_int((tid < n && pr > 0.0f && (double)r <= cum) ? tid : SMP_THREADS, ibuf);
            const int last = -block_min_int((tid < n && pr > 0.0f) ? -tid : 1, ibuf);
            if (first < SMP_THREADS) chosen = sort_i[first];
            else chosen = last >= 0 ? sort_i[last] : V - 1;
        } else {
        // ---- top-k in general: radix selection over the whole row ---------------------------
        if (a.top_k > 0 && a.top_k < V) {
            unsigned prefix = 0u, mask = 0u;

            int k_left = a.top_k;
            for (int shift = 24; shift >= 0; shift -= 8) {
                if (tid < 256) hist[tid] = 0u;
                __syncthreads();
#pragma unroll 8
                OWN_ROWS(j, i) {
                    if (i < V) {
                        const unsigned key = order_key(x[i]);
                        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
                    }
                }
                __syncthreads();
                if (tid == 0) {
                    int left = k_left;
                    int bin = 255;
                    for (; bin > 0; --bin) {
                        if ((int)hist[bin] >= left) break;
                        left -= (int)hist[bin];
                    }
                    sh_prefix = prefix | ((unsigned)bin << shift);
                    sh_int = left;
                }
                __syncthreads();
                prefix = sh_prefix;
                k_left = sh_int;
                mask |= 255u << shift;
                __syncthreads();
            }
            const float threshold = key_value(prefix);
#pragma unroll 8
            OWN_ROWS(j, i)
                if (i < V && x[i] < threshold) x[i] = -INFINITY;
            __syncthreads();
        }

        // ---- top-p over the softmax of the survivors ------------------------------------
        if (a.top_p > 0.0f && a.top_p < 1.0f) {
            int mine = 0;
            float mx_l = -INFINITY;
#pragma unroll 8
            OWN_ROWS(j, i) {
                if (i < V) {
                    const float v = x[i];
                    if (v > -INFINITY) { ++mine; mx_l = fmaxf(mx_l, v); }
                }
            }
            const int n_surv = block_sum_int(mine, ibuf);
            const float mx = block_max(mx_l, fscratch);
            if (n_surv > 0) {
                double part = 0.0;
#pragma unroll 8
                OWN_ROWS(j, i) {
                    if (i < V) {
                        const float v = x[i];
                        if (v > -INFINITY) part += exp((double)(v - mx));
                    }
                }
                const float sum_f = (float)block_sum_double(part, dbuf);
                if (n_surv <= SMP_SORT_MAX) {
                    // gather (in any order), sort by (probability descending, index ascending)
                    int sz = 32;
                    while (sz < n_surv) sz <<= 1;
                    if (tid < sz) { sort_p[tid] = -1.0f; sort_i[tid] = 0x7fffffff; }
                    if (tid == 0) sh_int = 0;
                    __syncthreads();
#pragma unroll 8
                    OWN_ROWS(j, i) {
                        if (i < V) {
                            const float v = x[i];
                            if (v > -INFINITY) {
                                const int at = atomicAdd(&sh_int, 1);
                                sort_p[at] = expf(v - mx) / sum_f;
                                sort_i[at] = i;
                            }
                        }
                    }
                    __syncthreads();
                    for (int size = 2; size <= sz; size <<= 1) {
                        for (int stride = size >> 1; stride > 0; stride >>= 1) {
                            if (tid < sz) {
                                const int partner = tid ^ stride;
                                if (partner > tid) {
                                    const bool descending_block = (tid & size) == 0;
                                    const float pa = sort_p[tid], pb = sort_p[partner];
                                    const int ia = sort_i[tid], ib = sort_i[partner];
                                    // "a before b" in the wanted order
                                    const bool a_first = pa > pb || (pa == pb && ia < ib);
                                    if (a_first != descending_block) {
                                        sort_p[tid] = pb; sort_p[partner] = pa;
                                        sort_i[tid] = ib; sort_i[partner] = ia;
                                    }
                                }
                            }
                            __syncthreads();
                        }
                    }
                    if (tid == 0) {
                        float cum = 0.0f;
                        int keep = n_surv;
                        for (int i = 0; i < n_surv; ++i) {
                            cum += sort_p[i];
                            if (cum > a.top_p) { keep = i + 1; break; }
                        }
                        sh_int = keep;
                    }
                    __syncthreads();
                    const int keep = sh_int;
                    for (int i = keep + tid; i < n_surv; i += SMP_THREADS) x[sort_i[i]] = -INFINITY;
                    __syncthreads();
                } else {
                    // too many survivors to sort: find the probability at which the running
                    // sum (descending) first exceeds p by radix selection over the float bits
                    unsigned prefix = 0u, mask = 0u;
                    double above = 0.0;                   // sum of probabilities above the prefix
                    for (int shift = 24; shift >= 0; shift -= 8) {
                        if (tid < 256) { hist[tid] = 0u; hsum[tid] = 0.0; }
                        __syncthreads();
                        OWN_ROWS(j, i) {
                            const float v = i < V ? x[i] : -INFINITY;
                            if (v > -INFINITY) {
                                const float pr = expf(v - mx) / sum_f;
                                const unsigned key = __float_as_uint(pr);
                                if ((key & mask) == prefix) {
                                    atomicAdd(&hist[(key >> shift) & 255u], 1u);
                                    atomicAdd(&hsum[(key >> shift) & 255u], (double)pr);
                                }
                            }
                        }
                        __syncthreads();
                        if (tid == 0) {
                            double run = above;
                            int bin = 255;
                            for (; bin > 0; --bin) {
                                if (hist[bin] != 0u && run + hsum[bin] > (double)a.top_p) break;
                                run += hsum[bin];
                            }
                            sh_prefix = prefix | ((unsigned)bin << shift);
                            sh_dbl = run;
                        }
                        __syncthreads();
                        prefix = sh_prefix;
                        above = sh_dbl;
                        mask |= 255u << shift;
                        __syncthreads();
                    }
                    // entries equal to the threshold: keep them in index order while needed
                    const float thr = __uint_as_float(prefix);
                    int ties = 0;
                    OWN_ROWS(j, i) {
                        const float v = i < V ? x[i] : -INFINITY;
                        if (v > -INFINITY && expf(v - mx) / sum_f == thr) ++ties;
                    }
                    // ties in the warps before this one
                    ties = warp_sum_int(ties);
                    if (lane == 0) ibuf[warp] = ties;
                    __syncthreads();
                    int rank = 0;
                    for (int w = 0; w < warp; ++w) rank += ibuf[w];
                    __syncthreads();
                    int need = 0x7fffffff;                // ties to keep
                    if (thr > 0.0f) {
                        const double gap = (double)a.top_p - above;
                        need = gap < 0.0 ? 1 : (int)floor(gap / (double)thr) + 1;
                    }
                    OWN_ROWS(j, i) {
                        const float v = i < V ? x[i] : -INFINITY;
                        const float pr = v > -INFINITY ? expf(v - mx) / sum_f : -1.0f;
                        const bool tie = pr == thr;
                        const unsigned tie_lanes = __ballot_sync(0xffffffffu, tie);
                        const int my_rank = rank + __popc(tie_lanes & ((1u << lane) - 1u));
                        if (v > -INFINITY && (pr < thr || (tie && my_rank >= need))) x[i] = -INFINITY;
                        rank += __popc(tie_lanes);
                    }
                    __syncthreads();
                }
            }
        }

        // ---- the draw ------------------------------------------------------------------
        const float inv_temp = 1.0f / a.temp;
        float mx_l = -INFINITY;
#pragma unroll 8
        OWN_ROWS(j, i)
            if (i < V) mx_l = fmaxf(mx_l, x[i] * inv_temp);
        const float mx = block_max(mx_l, fscratch);
        double part = 0.0;
#pragma unroll 8
        OWN_ROWS(j, i) {
            if (i < V) {
                const float v = x[i] * inv_temp;
                if (v > -INFINITY) part += (double)expf(v - mx);
            }
        }
        // each warp's share of the sum decides which warp's range holds the answer (the share
        // scaled by 1/sum stands for the sum of the range's float32 probabilities: they differ
        // in the eighth digit, and a draw that falls into that gap takes the range's last token)
        part = warp_sum_double(part);
        if (lane == 0) wsum[warp] = part;
        __syncthreads();
        double total = 0.0;
        for (int w = 0; w < 32; ++w) total += wsum[w];
        const float inv_sum = (float)(1.0 / total);
        __syncthreads();
        if (lane == 0) wsum[warp] = part * (double)inv_sum;
        __syncthreads();
        const unsigned draw = st ? (unsigned)st[1] : 0u;
        const unsigned stream = a.stream_ids ? (unsigned)a.stream_ids[row] : (unsigned)row;
        const float r = (float)(philox_uniform_bits(a.seed, draw, stream) >> 8) *
                        (1.0f / 16777216.0f);
        // the first warp whose running sum reaches r owns the answer
        double before = 0.0;
        int owner = 32;
        for (int w = 0; w < 32; ++w) {
            const double incl = before + wsum[w];
            if ((double)r <= incl && wsum[w] > 0.0) { owner = w; break; }
            before = incl;
        }
        auto prob = [&](int i) -> float {
            if (i >= V) return 0.0f;
            const float v = x[i] * inv_temp;
            return v > -INFINITY ? expf(v - mx) * inv_sum : 0.0f;
        };
        if (owner == 32) {
            if (tid == 0) sh_int = V - 1;                  // the reference's fallback
        } else {
            // all warps: the sums of the owner range's rows of 32 indices
            const int o_begin = owner * n_rows * 32;
            for (int rr = warp; rr < n_rows; rr += 32) {
                const double tot = warp_sum_double((double)prob(o_begin + rr * 32 + lane));
                if (lane == 0) rowtot[rr] = tot;
            }
            __syncthreads();
            if (warp == 0) {
                // the first row at which the running sum reaches r (32 rows at a time)
                double cum = before;
                int hit_row = -1, last_row = -1;
                double cum_at_row = 0.0;
                for (int g0 = 0; g0 < n_rows && hit_row < 0; g0 += 32) {
                    const int rr = g0 + lane;
                    const double tot = rr < n_rows ? rowtot[rr] : 0.0;
                    double run = tot;
#pragma unroll
                    for (int off = 1; off < 32; off <<= 1) {
                        const double up = __shfl_up_sync(0xffffffffu, run, off);
                        if (lane >= off) run += up;
                    }
                    const unsigned hits = __ballot_sync(0xffffffffu, tot > 0.0 && (double)r <= cum + run);
                    const unsigned live = __ballot_sync(0xffffffffu, tot > 0.0);
                    if (live != 0u) last_row = g0 + (31 - __clz(live));
                    if (hits != 0u) {
                        const int l = __ffs(hits) - 1;
                        hit_row = g0 + l;
                        cum_at_row = cum + __shfl_sync(0xffffffffu, run - tot, l);
                    }
                    cum += __shfl_sync(0xffffffffu, run, 31);
                }
                // inside that row (or, if rounding left none, the last row with mass)
                const int the_row = hit_row >= 0 ? hit_row : last_row;
                int pick = -1;
                if (the_row >= 0) {
                    const int i = o_begin + the_row * 32 + lane;
                    const float pr = prob(i);
                    double run = (double)pr;
#pragma unroll
                    for (int off = 1; off < 32; off <<= 1) {
                        const double up = __shfl_up_sync(0xffffffffu, run, off);
                        if (lane >= off) run += up;
                    }
                    const unsigned hits = __ballot_sync(0xffffffffu, hit_row >= 0 && pr > 0.0f && (double)r <= cum_at_row + run);
                    const unsigned live = __ballot_sync(0xffffffffu, pr > 0.0f);
                    if (hits != 0u) pick = i - lane + (__ffs(hits) - 1);
                    else if (live != 0u) pick = i - lane + (31 - __clz(live));
                }
                if (lane == 0) sh_int = pick >= 0 ? pick : V - 1;
            }
        }
        __syncthreads();
        chosen = sh_int;
        }   // the general path
    }
#undef OWN_ROWS

    if (tid == 0) {
        a.out[row] = chosen;
        if (st != nullptr && a.update_state) {
            st[2 + (st[0] % SMP_RECENT)] = chosen;
            st[0] += 1;
            st[1] += 1;
        }
    }
}

extern "C" int mf_sample(float* logits, long long ld, int rows, int vocab, const int* slots,
                         int* state, const int* stream_ids, int* out, float temp, int top_k,
                         float top_p, float repeat, float frequency, float presence,
                         unsigned long long seed, int update_state, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return MF_ERR_ARGUMENT;
    if ((vocab + SMP_THREADS - 1) / SMP_THREADS > SMP_THREADS) return MF_ERR_UNSUPPORTED;   // over 1,048,576
    SampleArgs a;
    a.logits = logits; a.ld = ld; a.vocab = vocab; a.slots = slots; a.state = state;
    a.stream_ids = stream_ids; a.out = out; a.temp = temp; a.top_k = top_k; a.top_p = top_p;
    a.repeat = repeat; a.frequency = frequency; a.presence = presence; a.seed = seed;
    a.update_state = update_state;
    mf_launch(sample_kernel, dim3(rows), dim3(SMP_THREADS), 0, stream, a);
    return MF_LAUNCH_CHECK();
}

extern "C" int mf_sampler_state_ints() { return SMP_STATE_INTS; }
