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
// depends on its neighbours.  The recent window and the draw counter live in a small
// fixed-size state per sequence: state[slot] = {n_seen, n_draws, ring[64]}.
#include "common.cuh"

#define SMP_THREADS 1024
#define SMP_RECENT 64
#define SMP_STATE_INTS (2 + SMP_RECENT)
#define SMP_SORT_MAX 1024

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

// inclusive scan of one double per thread over the block; returns this thread's inclusive sum
__device__ double block_scan_inclusive(double v, double* buf) {
    const int t = threadIdx.x;
    buf[t] = v;
    __syncthreads();
    for (int off = 1; off < SMP_THREADS; off <<= 1) {
        const double add = t >= off ? buf[t - off] : 0.0;
        __syncthreads();
        buf[t] += add;
        __syncthreads();
    }
    const double r = buf[t];
    __syncthreads();
    return r;
}
__device__ int block_scan_inclusive_int(int v, int* buf) {
    const int t = threadIdx.x;
    buf[t] = v;
    __syncthreads();
    for (int off = 1; off < SMP_THREADS; off <<= 1) {
        const int add = t >= off ? buf[t - off] : 0;
        __syncthreads();
        buf[t] += add;
        __syncthreads();
    }
    const int r = buf[t];
    __syncthreads();
    return r;
}
__device__ double block_sum_double(double v, double* buf) {
    const int t = threadIdx.x;
    buf[t] = v;
    __syncthreads();
    for (int off = SMP_THREADS / 2; off > 0; off >>= 1) {
        if (t < off) buf[t] += buf[t + off];
        __syncthreads();
    }
    const double r = buf[0];
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(SMP_THREADS) sample_kernel(SampleArgs a) {
    pdl_prologue();
    __shared__ double dbuf[SMP_THREADS];
    __shared__ float fscratch[33];
    __shared__ int ibuf[SMP_THREADS];
    __shared__ float sort_p[SMP_SORT_MAX];
    __shared__ int sort_i[SMP_SORT_MAX];
    __shared__ unsigned hist[256];
    __shared__ double hsum[256];
    __shared__ unsigned sh_prefix;
    __shared__ int sh_int;
    __shared__ double sh_dbl;

    const int row = blockIdx.x;
    const int tid = threadIdx.x;
    const int V = a.vocab;
    float* x = a.logits + (size_t)row * a.ld;
    int* st = (a.slots != nullptr && a.state != nullptr)
                  ? a.state + (size_t)a.slots[row] * SMP_STATE_INTS : nullptr;
    const int seg = (V + SMP_THREADS - 1) / SMP_THREADS;   // contiguous indices per thread
    const int i_begin = min(V, tid * seg), i_end = min(V, i_begin + seg);

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
        for (int i = i_begin; i < i_end; ++i) {
            const float v = x[i];
            if (best_i == V || v > best) { best = v; best_i = i; }
        }
        const float mx = block_max(best_i == V ? -INFINITY : best, fscratch);
        // lowest index among those equal to the maximum (a NaN row falls back to index 0)
        int cand = (best_i != V && best == mx) ? best_i : V;
        ibuf[tid] = cand;
        __syncthreads();
        for (int off = SMP_THREADS / 2; off > 0; off >>= 1) {
            if (tid < off) ibuf[tid] = min(ibuf[tid], ibuf[tid + off]);
            __syncthreads();
        }
        chosen = ibuf[0] < V ? ibuf[0] : 0;
        __syncthreads();
    } else {
        // ---- top-k: mask everything below the k-th largest value ------------------------
        if (a.top_k > 0 && a.top_k < V) {
            unsigned prefix = 0u, mask = 0u;
            int k_left = a.top_k;
            for (int shift = 24; shift >= 0; shift -= 8) {
                if (tid < 256) hist[tid] = 0u;
                __syncthreads();
                for (int i = tid; i < V; i += SMP_THREADS) {
                    const unsigned key = order_key(x[i]);
                    if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
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
            for (int i = tid; i < V; i += SMP_THREADS)
                if (x[i] < threshold) x[i] = -INFINITY;
            __syncthreads();
        }

        // ---- top-p over the softmax of the survivors ------------------------------------
        if (a.top_p > 0.0f && a.top_p < 1.0f) {
            int mine = 0;
            float mx_l = -INFINITY;
            for (int i = i_begin; i < i_end; ++i) {
                const float v = x[i];
                if (v > -INFINITY) { ++mine; mx_l = fmaxf(mx_l, v); }
            }
            const int incl = block_scan_inclusive_int(mine, ibuf);
            if (tid == SMP_THREADS - 1) sh_int = incl;
            __syncthreads();
            const int n_surv = sh_int;
            const float mx = block_max(mx_l, fscratch);
            if (n_surv > 0) {
                double part = 0.0;
                for (int i = i_begin; i < i_end; ++i) {
                    const float v = x[i];
                    if (v > -INFINITY) part += exp((double)(v - mx));
                }
                const float sum_f = (float)block_sum_double(part, dbuf);
                if (n_surv <= SMP_SORT_MAX) {
                    // gather in index order, sort by (probability descending, index ascending)
                    if (tid < SMP_SORT_MAX) { sort_p[tid] = -1.0f; sort_i[tid] = 0x7fffffff; }
                    __syncthreads();
                    int at = incl - mine;
                    for (int i = i_begin; i < i_end; ++i) {
                        const float v = x[i];
                        if (v > -INFINITY) { sort_p[at] = expf(v - mx) / sum_f; sort_i[at] = i; ++at; }
                    }
                    __syncthreads();
                    for (int size = 2; size <= SMP_SORT_MAX; size <<= 1) {
                        for (int stride = size >> 1; stride > 0; stride >>= 1) {
                            if (tid < SMP_SORT_MAX) {
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
                        for (int i = tid; i < V; i += SMP_THREADS) {
                            const float v = x[i];
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
                    for (int i = i_begin; i < i_end; ++i) {
                        const float v = x[i];
                        if (v > -INFINITY && expf(v - mx) / sum_f == thr) ++ties;
                    }
                    int rank = block_scan_inclusive_int(ties, ibuf) - ties;
                    int need = 0x7fffffff;                // ties to keep
                    if (thr > 0.0f) {
                        const double gap = (double)a.top_p - above;
                        need = gap < 0.0 ? 1 : (int)floor(gap / (double)thr) + 1;
                    }
                    for (int i = i_begin; i < i_end; ++i) {
                        const float v = x[i];
                        if (v > -INFINITY) {
                            const float pr = expf(v - mx) / sum_f;
                            if (pr < thr) x[i] = -INFINITY;
                            else if (pr == thr) { if (rank >= need) x[i] = -INFINITY; ++rank; }
                        }
                    }
                    __syncthreads();
                }
            }
        }

        // ---- the draw ------------------------------------------------------------------
        const float inv_temp = 1.0f / a.temp;
        float mx_l = -INFINITY;
        for (int i = i_begin; i < i_end; ++i) mx_l = fmaxf(mx_l, x[i] * inv_temp);
        const float mx = block_max(mx_l, fscratch);
        double part = 0.0;
        for (int i = i_begin; i < i_end; ++i) {
            const float v = x[i] * inv_temp;
            if (v > -INFINITY) part += (double)expf(v - mx);
        }
        const double total = block_sum_double(part, dbuf);
        const float inv_sum = (float)(1.0 / total);
        double mine = 0.0;
        for (int i = i_begin; i < i_end; ++i) {
            const float v = x[i] * inv_temp;
            if (v > -INFINITY) mine += (double)(expf(v - mx) * inv_sum);
        }
        const double incl = block_scan_inclusive(mine, dbuf);
        const unsigned draw = st ? (unsigned)st[1] : 0u;
        const unsigned stream = a.stream_ids ? (unsigned)a.stream_ids[row] : (unsigned)row;
        const float r = (float)(philox_uniform_bits(a.seed, draw, stream) >> 8) *
                        (1.0f / 16777216.0f);
        // the first thread whose inclusive sum reaches r owns the answer
        ibuf[tid] = ((double)r <= incl && mine > 0.0) ? tid : SMP_THREADS;
        __syncthreads();
        for (int off = SMP_THREADS / 2; off > 0; off >>= 1) {
            if (tid < off) ibuf[tid] = min(ibuf[tid], ibuf[tid + off]);
            __syncthreads();
        }
        const int owner = ibuf[0];
        __syncthreads();
        if (owner == SMP_THREADS) {
            if (tid == 0) sh_int = V - 1;                  // the reference's fallback
        } else if (tid == owner) {
            double cum = incl - mine;
            int pick = -1, last_pos = -1;
            for (int i = i_begin; i < i_end; ++i) {
                const float v = x[i] * inv_temp;
                if (!(v > -INFINITY)) continue;
                const float pr = expf(v - mx) * inv_sum;
                if (pr <= 0.0f) continue;
                cum += (double)pr;
                last_pos = i;
                if ((double)r <= cum) { pick = i; break; }
            }
            sh_int = pick >= 0 ? pick : last_pos;
        }
        __syncthreads();
        chosen = sh_int;
    }

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
    SampleArgs a;
    a.logits = logits; a.ld = ld; a.vocab = vocab; a.slots = slots; a.state = state;
    a.stream_ids = stream_ids; a.out = out; a.temp = temp; a.top_k = top_k; a.top_p = top_p;
    a.repeat = repeat; a.frequency = frequency; a.presence = presence; a.seed = seed;
    a.update_state = update_state;
    mf_launch(sample_kernel, dim3(rows), dim3(SMP_THREADS), 0, stream, a);
    return MF_LAUNCH_CHECK();
}

extern "C" int mf_sampler_state_ints() { return SMP_STATE_INTS; }
