// out[M,N] = epilogue(x[M,K] . W[N,K]^T + bias[N]) for a handful of rows (M <= 16): decoding.
//
// With so few rows the product is a stream of the weight matrix from HBM, so the kernel is
// built around that stream. The roles are swapped with respect to the usual layout: 16
// weight rows (output features) are the M side of mma.sync.m16n8k16 and the tokens are its
// N side (8 per MMA, one or two blocks). A block of eight warps owns 16 output features;
// warp w takes the 32-wide blocks of K numbered w, w + 8, ..., so that at any moment the
// block reads adjacent pieces of the same 16 rows. Every thread reads 16 contiguous bytes of
// a weight row and of an activation row per block (the contraction order is permuted the
// same way on both sides: thread t of a quad takes dims 8t..8t+7), keeps eight weight
// loads in flight, and accumulates in float. The eight warps' partial sums are added in a
// fixed order through shared memory, then bias / GELU / residual are applied and the
// result is stored: no separate epilogue pass, and a row's result does not depend on the
// other rows of the batch. The reference runs these products through nn.Linear
// (app/architectures/qwen_layers.py:50-53, app/architectures/starcoder2_layers.py:19-23).
//
// Epilogue modes as in gemm_simt.cu: 0 out(bf16) = v; 1 out(bf16) = gelu_tanh(v);
// 2 out(f32) = residual + v; 3 out(f32) = v, with v = acc + bias.
#include "common.cuh"

namespace {

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_UNROLL = 4;

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2,
                                               unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_stream(const __nv_bfloat16* p) {
    // weights are read once per step: keep them from displacing the activations in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int MB>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ W,
                   int ldw, const float* __restrict__ bias, const float* residual, void* out,
                   int ldo, int M, int N, int K, int mode) {
    __shared__ float red[SK_WARPS][16][8 * MB];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    const bool row_ok[2] = {n0 + g < N, n0 + g + 8 < N};
    const __nv_bfloat16* wrow[2] = {W + (size_t)min(n0 + g, N - 1) * ldw + 8 * t,
                                    W + (size_t)min(n0 + g + 8, N - 1) * ldw + 8 * t};
    const __nv_bfloat16* xrow[MB];
    bool tok_ok[MB];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        tok_ok[mb] = 8 * mb + g < M;
        xrow[mb] = x + (size_t)min(8 * mb + g, M - 1) * ldx + 8 * t;
    }
    float acc[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) acc[mb][0] = acc[mb][1] = acc[mb][2] = acc[mb][3] = 0.f;

    const int n_blocks = K / 32;
    // The weights are nobody's output: start pulling this thread's first pieces towards L2 while
    // the kernel before this one is still finishing, then wait for it before touching activations.
    pdl_trigger();
#pragma unroll
    for (int u = 0; u < 2 * SK_UNROLL; ++u) {
        const int kb = warp + u * SK_WARPS;
        if (kb < n_blocks) {
            if (row_ok[0]) prefetch_l2(wrow[0] + 32 * kb);
            if (row_ok[1]) prefetch_l2(wrow[1] + 32 * kb);
        }
    }
    pdl_wait();
    for (int kb0 = warp; kb0 < n_blocks; kb0 += SK_WARPS * SK_UNROLL) {
        uint4 wf[SK_UNROLL][2], xf[SK_UNROLL][MB];
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u) {
            const int kb = kb0 + u * SK_WARPS;
            const bool in = kb < n_blocks;
#pragma unroll
            for (int i = 0; i < 2; ++i)
                wf[u][i] = (in && row_ok[i]) ? load_stream(wrow[i] + 32 * kb) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
                xf[u][mb] = (in && tok_ok[mb]) ? *reinterpret_cast<const uint4*>(xrow[mb] + 32 * kb)
                                               : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u)
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                mma_bf16_16816(acc[mb], wf[u][0].x, wf[u][1].x, wf[u][0].y, wf[u][1].y, xf[u][mb].x, xf[u][mb].y);
                mma_bf16_16816(acc[mb], wf[u][0].z, wf[u][1].z, wf[u][0].w, wf[u][1].w, xf[u][mb].z, xf[u][mb].w);
            }
    }
    // this thread holds features g, g + 8 for tokens 8 mb + 2t, + 1
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        red[warp][g][8 * mb + 2 * t] = acc[mb][0];
        red[warp][g][8 * mb + 2 * t + 1] = acc[mb][1];
        red[warp][g + 8][8 * mb + 2 * t] = acc[mb][2];
        red[warp][g + 8][8 * mb + 2 * t + 1] = acc[mb][3];
    }
    __syncthreads();
    for (int idx = tid; idx < 16 * 8 * MB; idx += SK_THREADS) {
        const int f = idx & 15, m = idx >> 4;
        const int n = n0 + f;
        if (n >= N || m >= M) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) v += red[w][f][m];
        if (bias) v += bias[n];
        if (mode == 1) v = gelu_tanh_fast(v);
        const size_t o = (size_t)m * ldo + n;
        if (mode >= 2) {
            if (mode == 2) v += residual[o];
            reinterpret_cast<float*>(out)[o] = v;
        } else {
            reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
        }
    }
}

}  // namespace

extern "C" int mx_gemm_skinny(const void* x, const void* W, const float* bias, const float* residual,
                              void* out, int out_dtype, int M, int N, int K, int ldx, int ldw, int ldo,
                              int mode, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return MX_OK;
    if (M > 16) MX_REFUSE("skinny gemm: %d rows, this kernel takes at most 16", M);
    if (K <= 0 || K % 32 != 0) MX_REFUSE("skinny gemm: K = %d is not a positive multiple of 32", K);
    if (ldx % 8 != 0 || ldw % 8 != 0) MX_REFUSE("skinny gemm: row strides %d, %d are not multiples of 8", ldx, ldw);
    if (mode < 0 || mode > 3) MX_REFUSE("skinny gemm: unknown epilogue mode %d", mode);
    if (mode == 2 && residual == nullptr) MX_REFUSE("skinny gemm: residual mode without a residual");
    if ((mode >= 2) != (out_dtype == MX_DTYPE_F32))
        MX_REFUSE("skinny gemm: epilogue mode %d does not write dtype %d", mode, out_dtype);
    const int grid = (N + 15) / 16;
    if (M <= 8)
        mx_launch_chained(gemm_skinny_kernel<1>, dim3(grid), dim3(SK_THREADS), 0, stream,
                          (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)W, ldw, bias, residual, out, ldo,
                          M, N, K, mode);
    else
        mx_launch_chained(gemm_skinny_kernel<2>, dim3(grid), dim3(SK_THREADS), 0, stream,
                          (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)W, ldw, bias, residual, out, ldo,
                          M, N, K, mode);
    return mx_launch_status();
}
