// C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores, 32-bit accumulation, any M, N, K.
//
// This is the matrix product of the true 32-bit path (no tensor cores, so no
// reduced-precision matrix mode), and the fallback of the bfloat16 path for
// shapes that the tensor-core kernel refuses.  Every output element is summed
// by one thread over k ascending with fused multiply-adds, so its value does
// not depend on M, on the tile it falls into, or on the rest of the batch.
// It restates the reference's row-times-vector product (infer/matmul.odin:63-70)
// for many rows of A at once.
#include "common.cuh"

#define TM 64
#define TN 64
#define TK 16

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_plain_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                         TC* __restrict__ C, int M, int N, int K, size_t lda,
                                                         size_t ldw, size_t ldc) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Ws[TK][TN + 4];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    const int lrow = tid >> 2;        // 0..63
    const int lk = (tid & 3) * 4;     // 0,4,8,12
    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int m = m0 + lrow, n = n0 + lrow;
            As[lk + i][lrow] = (m < M && k < K) ? to_f32(A[(size_t)m * lda + k]) : 0.f;
            Ws[lk + i][lrow] = (n < N && k < K) ? to_f32(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
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
            if (n < N) C[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
        }
    }
}

// Element types: a_dtype of A, w_dtype of W, c_dtype of C.  Leading dimensions
// in elements.
extern "C" int odin_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                               int M, int N, int K, long long lda, long long ldw, long long ldc,
                               void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    if (grid.y > 65535) return ODIN_ERR_UNSUPPORTED;
#define GO(TA, TW, TC)                                                                                     \
    odin_launch(gemm_plain_kernel<TA, TW, TC>, grid, dim3(256), 0, s, (const TA*)A, (const TW*)W, (TC*)C, M, N, K, \
                (size_t)lda, (size_t)ldw, (size_t)ldc)
    const int key = a_dtype * 4 + w_dtype * 2 + c_dtype;
    switch (key) {
        case 0: GO(float, float, float); break;
        case 1: GO(float, float, bf16); break;
        case 2: GO(float, bf16, float); break;
        case 3: GO(float, bf16, bf16); break;
        case 4: GO(bf16, float, float); break;
        case 5: GO(bf16, float, bf16); break;
        case 6: GO(bf16, bf16, float); break;
        case 7: GO(bf16, bf16, bf16); break;
        default: return ODIN_ERR_UNSUPPORTED;
    }
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}
