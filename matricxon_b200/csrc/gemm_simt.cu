// out[M,N] = epilogue(A[M,K] . W[N,K]^T + bias[N]) on the FP32 cores.
//
// This is the true 32-bit matrix product of the engine (inputs, products and sums are
// float; no tensor-core mode), and the plain twin that the tensor-core product is checked
// against. Each output element is one fixed-order sum over K, whatever M is, so a row's
// result does not depend on what else is in the batch. The reference runs these products
// through nn.Linear (app/architectures/qwen_layers.py:50-53,
// app/architectures/starcoder2_layers.py:19-23).
//
// Epilogue modes: 0 out(T) = v; 1 out(T) = gelu_tanh(v); 2 out(f32) = residual + v;
// 3 out(f32) = v, where v = acc + bias.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int THREADS = (BM / TM) * (BN / TN);  // 256

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const TIn* __restrict__ A, const TIn* __restrict__ W,
                 const float* __restrict__ bias, const float* residual, TOut* out,
                 int M, int N, int K, int lda, int ldw, int ldo, int mode) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // each thread stages 4 elements of A and 4 of W per k-tile: row = tid / 4, 4 k's at (tid % 4) * 4
    const int lrow = tid >> 2, lk = (tid & 3) << 2;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + e][lrow] = (am < M && k < K) ? to_float(A[(size_t)am * lda + k]) : 0.f;
            Ws[lk + e][lrow] = (wn < N && k < K) ? to_float(W[(size_t)wn * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            if (mode == 1) v = gelu_tanh(v);
            const size_t o = (size_t)m * ldo + n;
            if (mode == 2) v += residual[o];
            out[o] = from_float<TOut>(v);
        }
    }
}

}  // namespace

extern "C" int mx_gemm_simt(const void* A, const void* W, int in_dtype, const float* bias,
                            const float* residual, void* out, int out_dtype, int M, int N, int K,
                            int lda, int ldw, int ldo, int mode, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return MX_OK;
    if (K <= 0) MX_REFUSE("gemm: K must be positive, got %d", K);
    if (mode < 0 || mode > 3) MX_REFUSE("gemm: unknown epilogue mode %d", mode);
    if (mode == 2 && residual == nullptr) MX_REFUSE("gemm: residual mode without a residual");
    const int expected_out = (mode >= 2 || in_dtype == MX_DTYPE_F32) ? MX_DTYPE_F32 : MX_DTYPE_BF16;
    if (out_dtype != expected_out)
        MX_REFUSE("gemm: epilogue mode %d with input dtype %d writes dtype %d, not %d", mode,
                  in_dtype, expected_out, out_dtype);
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) MX_REFUSE("gemm: M = %d is beyond this kernel's grid", M);
#define MX_GEMM(TI, TO) \
    gemm_simt_kernel<TI, TO><<<grid, THREADS, 0, stream>>>((const TI*)A, (const TI*)W, bias, residual, (TO*)out, M, N, K, lda, ldw, ldo, mode)
    if (in_dtype == MX_DTYPE_F32 && out_dtype == MX_DTYPE_F32) MX_GEMM(float, float);
    else if (in_dtype == MX_DTYPE_BF16 && out_dtype == MX_DTYPE_F32) MX_GEMM(__nv_bfloat16, float);
    else if (in_dtype == MX_DTYPE_BF16 && out_dtype == MX_DTYPE_BF16) MX_GEMM(__nv_bfloat16, __nv_bfloat16);
    else MX_REFUSE("gemm: float inputs with a bfloat16 output are not used by any path");
#undef MX_GEMM
    return mx_launch_status();
}
