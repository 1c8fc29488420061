// Plain matrix product on the FP32 pipe: C[M][N] (+)= A[M][K] * W[N][K]^T + bias[N].
//
// This is the true 32-bit path of every projection (FFMA only, no tensor-core mode, so no
// TF32 or bfloat16 staging) and the twin that the tensor-core kernels are checked against.
// Weights are [out][in] row-major and activations token-major as in the reference
// (src/graph/ops.rs:132-136; out[t*od+o] = dot(w[o], x[t]) + bias[o],
// src/graph/cpu_backend.rs:214-247).
//
// Each output element is summed over k in ascending order by one thread, whatever M is and
// wherever the row lies in the batch, so a token's result never depends on its neighbours.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

// accumulate: 0  C = acc + bias        1  C = C + acc + bias  (C float32: residual stream)
template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias,
                 TC* __restrict__ C, int M, int N, int K, long long lda, long long ldw,
                 long long ldc, int accumulate) {
    pdl_prologue();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k per operand = 1024 elements, 4 per thread; k fastest for coalescing
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            float a = 0.0f, w = 0.0f;
            if (k < K) {
                if (m0 + r < M) a = to_f32(A[(size_t)(m0 + r) * lda + k]);
                if (n0 + r < N) w = to_f32(W[(size_t)(n0 + r) * ldw + k]);
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            TC* c = C + (size_t)m * ldc + n;
            if (accumulate) v += to_f32(*c);
            *c = from_f32<TC>(v);
        }
    }
}

extern "C" int mf_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype,
                            const float* bias, void* C, int c_dtype, int M, int N, int K,
                            long long lda, long long ldw, long long ldc, int accumulate,
                            cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return MF_ERR_ARGUMENT;
    if (accumulate && c_dtype != MF_DTYPE_F32) return MF_ERR_UNSUPPORTED;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return MF_ERR_UNSUPPORTED;
#define MF_GEMM(TA, TW, TC)                                                                  \
    mf_launch(gemm_simt_kernel<TA, TW, TC>, dim3(grid), dim3(256), 0, stream, (const TA*)A, (const TW*)W, bias,  \
                                                           (TC*)C, M, N, K, lda, ldw, ldc,   \
                                                           accumulate)
    typedef __nv_bfloat16 bf16;
    const int key = a_dtype * 4 + w_dtype * 2 + c_dtype;
    switch (key) {
        case 0: MF_GEMM(float, float, float); break;
        case 1: MF_GEMM(float, float, bf16); break;
        case 2: MF_GEMM(float, bf16, float); break;
        case 3: MF_GEMM(float, bf16, bf16); break;
        case 4: MF_GEMM(bf16, float, float); break;
        case 5: MF_GEMM(bf16, float, bf16); break;
        case 6: MF_GEMM(bf16, bf16, float); break;
        case 7: MF_GEMM(bf16, bf16, bf16); break;
        default: return MF_ERR_UNSUPPORTED;
    }
#undef MF_GEMM
    return MF_LAUNCH_CHECK();
}
