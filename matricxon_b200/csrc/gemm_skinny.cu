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
#include <cooperative_groups.h>

#include "common.cuh"

namespace {

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_UNROLL = 4;
constexpr int SK_DEEP = 6;      // K = 3,072 is then two trips to memory per warp instead of three

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2,
                                               unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 32 bytes at once (sm_100 has 256-bit loads): four lanes then cover a whole 128-byte line of a weight row,
// and a warp's load is eight whole lines instead of eight halves. The address must be 32-byte aligned.
__device__ __forceinline__ void load_stream32(const __nv_bfloat16* p, uint4& lo, uint4& hi) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
                 : "l"(p));
}

__device__ __forceinline__ uint4 load_stream(const __nv_bfloat16* p) {
    // weights are read once per step: keep them from displacing the activations in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Rotation and cache write in the epilogue of the QKV product (ROPE kernels): tile u of a rotated
// head (a query or key head) holds dims 8j..8j+7 as its rows 0-7 and their partners at
// + head_dim / 2 as rows 8-15, so the pair of every rotation is in one block; value heads keep 16
// consecutive dims. Queries go to `out` (the qkv buffer, row stride ldo), rotated keys and the
// values to their slot of the paged cache: what mx_rope_kv_write does after a plain product
// (app/architectures/rope.py:152-169, app/architectures/qwen_layers.py:80-86).
struct SkinnyRope {
    const int* positions;
    const float* inv_freq;          // [head_dim / 2]
    const int* slots;               // may be null: nothing is stored
    __nv_bfloat16* cache;           // [page][2][kv head][page_size * head_dim], keys [slot][dim], values [dim][slot]
    int* status;
    long long n_slots;
    int n_heads, n_kv_heads, head_dim, page_size;
};

// SPLIT: two blocks (a cluster of two, rank = blockIdx.x & 1) share a tile and take half of K each;
// the second hands its sums to the first through distributed shared memory, which adds them after its
// own (a fixed order) and runs the epilogue. For matrices with so few output features that one block
// per tile leaves most of the GPU's warp slots, and so most of the loads it could have in flight, unused.
template <int MB, bool ROPE, bool SPLIT, int UNROLL = SK_UNROLL, bool WIDE = false>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ W,
                   int ldw, const float* __restrict__ bias, const float* residual, void* out,
                   int ldo, int M, int N, int K, int mode, const SkinnyRope rope) {
    // UNROLL: weight loads in flight per thread = 2 UNROLL. Eight (the default) is best where an SM has three
    // blocks to run (sixteen measured slower there); products with at most two blocks an SM take SK_DEEP.
    constexpr int ROWS = 16, NR = 2;                   // a block owns 16 output features: rows g and g + 8 per thread
    __shared__ float red[SK_WARPS][ROWS][8 * MB];
    __shared__ float peer[SPLIT ? ROWS : 1][8 * MB];   // SPLIT: the other block's sums, written by it
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tile = SPLIT ? blockIdx.x >> 1 : blockIdx.x;
    const int half = SPLIT ? blockIdx.x & 1 : 0;
    int n_row[2];
    if (ROPE) {
        const int per_head = rope.head_dim >> 4;
        const int head = blockIdx.x / per_head, j = blockIdx.x - head * per_head;
        const bool rotated = head < rope.n_heads + rope.n_kv_heads;
        n_row[0] = head * rope.head_dim + (rotated ? 8 * j : 16 * j) + g;
        n_row[1] = n_row[0] + (rotated ? rope.head_dim / 2 : 8);
    } else {
        n_row[0] = tile * ROWS + g;
        n_row[1] = n_row[0] + 8;
    }
    bool row_ok[NR];
    const __nv_bfloat16* wrow[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        row_ok[i] = n_row[i] < N;
        wrow[i] = W + (size_t)min(n_row[i], N - 1) * ldw + (WIDE ? 16 : 8) * t;
    }
    const __nv_bfloat16* xrow[MB];
    bool tok_ok[MB];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        tok_ok[mb] = 8 * mb + g < M;
        xrow[mb] = x + (size_t)min(8 * mb + g, M - 1) * ldx + (WIDE ? 16 : 8) * t;
    }
    float acc[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) acc[mb][0] = acc[mb][1] = acc[mb][2] = acc[mb][3] = 0.f;

    // a piece of K is 32 elements per row (16 bytes a thread), or 64 with 32-byte loads (WIDE, never with SPLIT)
    constexpr int PIECE = WIDE ? 64 : 32, HALVES = WIDE ? 2 : 1;
    const int kb_first = SPLIT ? half * (K / 64) : 0;          // SPLIT needs K to be a multiple of 64
    const int n_blocks = SPLIT ? kb_first + K / 64 : K / PIECE;
    // The weights are nobody's output: start pulling this thread's first pieces towards L2 while
    // the kernel before this one is still finishing, then wait for it before touching activations.
#ifndef SK_PREFETCH_ITERS
#define SK_PREFETCH_ITERS 4     // one to eight measured alike, none and twelve or more slower
#endif
#pragma unroll
    for (int u = 0; u < SK_PREFETCH_ITERS; ++u) {
        const int kb = kb_first + warp + u * SK_WARPS;
        if (kb < n_blocks) {
#pragma unroll
            for (int i = 0; i < NR; ++i)
                if (row_ok[i]) prefetch_l2(wrow[i] + PIECE * kb);
        }
    }
    pdl_wait();
    // the activations (and the residual) are what the kernels before wrote: their pointers are taken anew
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) xrow[mb] = after_wait(xrow[mb]);
    residual = after_wait(residual);
    for (int kb0 = kb_first + warp; kb0 < n_blocks; kb0 += SK_WARPS * UNROLL) {
        uint4 wf[UNROLL][2][HALVES], xf[UNROLL][MB][HALVES];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int kb = kb0 + u * SK_WARPS;
            const bool in = kb < n_blocks;
#pragma unroll
            for (int i = 0; i < NR; ++i) {
#pragma unroll
                for (int h = 0; h < HALVES; ++h) wf[u][i][h] = make_uint4(0, 0, 0, 0);
                if (in && row_ok[i]) {
                    if constexpr (WIDE) load_stream32(wrow[i] + PIECE * kb, wf[u][i][0], wf[u][i][HALVES - 1]);
                    else wf[u][i][0] = load_stream(wrow[i] + PIECE * kb);
                }
            }
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
                    xf[u][mb][h] = (in && tok_ok[mb]) ? *reinterpret_cast<const uint4*>(xrow[mb] + PIECE * kb + 8 * h)
                                                      : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    mma_bf16_16816(acc[mb], wf[u][0][h].x, wf[u][1][h].x, wf[u][0][h].y, wf[u][1][h].y, xf[u][mb][h].x,
                                   xf[u][mb][h].y);
                    mma_bf16_16816(acc[mb], wf[u][0][h].z, wf[u][1][h].z, wf[u][0][h].w, wf[u][1][h].w, xf[u][mb][h].z,
                                   xf[u][mb][h].w);
                }
    }
    // All of this block's weights are on their way: the next kernel may start its own preamble (its
    // weights' first pieces towards L2) under this kernel's reduction and epilogue. Triggering at the top
    // instead lets the whole chain of kernels pile up behind the one that runs, each asking for its
    // weights at once (a decode step of 8 rows: 2.175 ms against 2.127 ms this way, 2.155 ms unchained).
    pdl_trigger();
    // this thread holds features g (and g + 8) for tokens 8 mb + 2t, + 1
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        red[warp][g][8 * mb + 2 * t] = acc[mb][0];
        red[warp][g][8 * mb + 2 * t + 1] = acc[mb][1];
        if (ROWS == 16) {
            red[warp][(g + 8) % ROWS][8 * mb + 2 * t] = acc[mb][2];
            red[warp][(g + 8) % ROWS][8 * mb + 2 * t + 1] = acc[mb][3];
        }
    }
    __syncthreads();
    auto total = [&](int f, int m) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) v += red[w][f][m];
        if (SPLIT) v += peer[SPLIT ? f : 0][m];
        return v;
    };
    if constexpr (SPLIT) {
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        if (half == 1) {
            float* remote = cluster.map_shared_rank(&peer[0][0], 0);
            for (int idx = tid; idx < ROWS * 8 * MB; idx += SK_THREADS) {
                const int f = idx % ROWS, m = idx / ROWS;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < SK_WARPS; ++w) v += red[w][f][m];
                remote[f * 8 * MB + m] = v;
            }
        }
        cluster.sync();
        if (half == 1) return;
    }
    if constexpr (ROPE) {
        const int HD = rope.head_dim;
        const int per_head = HD >> 4;
        const int head = blockIdx.x / per_head, j = blockIdx.x - head * per_head;
        const bool rotated = head < rope.n_heads + rope.n_kv_heads;
        const int m = rotated ? tid >> 3 : tid >> 4;
        if (tid >= (rotated ? 8 : 16) * 8 * MB || m >= M) return;
        long long page = 0;
        int offset = 0;
        if (head >= rope.n_heads) {          // a key or value head: the slot of this row's token
            if (rope.slots == nullptr) return;
            const long long slot = rope.slots[m];
            if (slot == -1) return;          // a padding row of a fixed-size batch
            if (slot < 0 || slot >= rope.n_slots) {
                atomicOr(rope.status, MX_STATUS_BAD_SLOT);
                return;
            }
            page = slot / rope.page_size;
            offset = (int)(slot - page * rope.page_size);
        }
        const size_t head_stride = (size_t)rope.page_size * HD;
        if (rotated) {
            const int i = tid & 7;
            const int d_lo = 8 * j + i, d_hi = d_lo + HD / 2;
            float lo = total(i, m), hi = total(i + 8, m);
            if (bias) {
                lo += bias[head * HD + d_lo];
                hi += bias[head * HD + d_hi];
            }
            // a plain product would round to bfloat16 before the rotation reads it: the same here
            lo = __bfloat162float(__float2bfloat16_rn(lo));
            hi = __bfloat162float(__float2bfloat16_rn(hi));
            const float angle = (float)rope.positions[m] * rope.inv_freq[d_lo];
            const float c = cosf(angle), sn = sinf(angle);
            __nv_bfloat16* dst = head < rope.n_heads
                                     ? reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * ldo + (size_t)head * HD
                                     : rope.cache + ((size_t)page * 2 * rope.n_kv_heads + (head - rope.n_heads)) * head_stride +
                                           (size_t)offset * HD;
            dst[d_lo] = __float2bfloat16_rn(lo * c - hi * sn);
            dst[d_hi] = __float2bfloat16_rn(hi * c + lo * sn);
        } else {
            const int r = tid & 15;
            const int dim = 16 * j + r;
            float v = total(r, m);
            if (bias) v += bias[head * HD + dim];
            rope.cache[((size_t)page * 2 * rope.n_kv_heads + rope.n_kv_heads + (head - rope.n_heads - rope.n_kv_heads)) *
                           head_stride + (size_t)dim * rope.page_size + offset] = __float2bfloat16_rn(v);
        }
    } else {
    for (int idx = tid; idx < ROWS * 8 * MB; idx += SK_THREADS) {
        const int f = idx % ROWS, m = idx / ROWS;
        const int n = tile * ROWS + f;
        if (n >= N || m >= M) continue;
        float v = total(f, m);
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
}

int skinny_sm_count() {
    static int count = 0;
    if (count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
        if (count <= 0) count = 148;
    }
    return count;
}

// Few blocks (at most two an SM) with more than one trip to memory each: more loads in flight per thread,
// at the price of registers that such a product does not need for a third block.
bool skinny_deep(int grid, int K) {
    return grid <= 2 * skinny_sm_count() && K / 32 > SK_WARPS * SK_UNROLL;
}

// 32-byte loads want pieces of 64 and rows that start on 32-byte boundaries
bool skinny_wide_ok(const void* W, int K, int ldw) {
    return K % 64 == 0 && ldw % 16 == 0 && reinterpret_cast<uintptr_t>(W) % 32 == 0;
}

int check_skinny(int M, int K, int ldx, int ldw) {
    if (M > 16) MX_REFUSE("skinny gemm: %d rows, this kernel takes at most 16", M);
    if (K <= 0 || K % 32 != 0) MX_REFUSE("skinny gemm: K = %d is not a positive multiple of 32", K);
    if (ldx % 8 != 0 || ldw % 8 != 0) MX_REFUSE("skinny gemm: row strides %d, %d are not multiples of 8", ldx, ldw);
    return MX_OK;
}

}  // namespace

extern "C" int mx_gemm_skinny(const void* x, const void* W, const float* bias, const float* residual,
                              void* out, int out_dtype, int M, int N, int K, int ldx, int ldw, int ldo,
                              int mode, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return MX_OK;
    const int rc = check_skinny(M, K, ldx, ldw);
    if (rc != MX_OK) return rc;
    if (mode < 0 || mode > 3) MX_REFUSE("skinny gemm: unknown epilogue mode %d", mode);
    if (mode == 2 && residual == nullptr) MX_REFUSE("skinny gemm: residual mode without a residual");
    if ((mode >= 2) != (out_dtype == MX_DTYPE_F32))
        MX_REFUSE("skinny gemm: epilogue mode %d does not write dtype %d", mode, out_dtype);
    const SkinnyRope none = {};
    const int grid = (N + 15) / 16;
    if (2 * grid <= 3 * skinny_sm_count() && K % 64 == 0 && K >= 6144) {
        // few tiles and a long K: two blocks a tile, as a cluster of two (c_proj 3072 x 12288: 14.8 us
        // against 16.9; at K = 3072 the halves are too short to pay for the exchange: 6.7 against 6.6)
        auto kernel = M <= 8 ? gemm_skinny_kernel<1, false, true> : gemm_skinny_kernel<2, false, true>;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(2 * grid);
        config.blockDim = dim3(SK_THREADS);
        config.stream = stream;
        cudaLaunchAttribute attribute[2];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = 2;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[1].val.programmaticStreamSerializationAllowed = mx_chained_launch_enabled() ? 1 : 0;
        config.attrs = attribute;
        config.numAttrs = 2;
        const cudaError_t e = cudaLaunchKernelEx(&config, kernel, (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)W,
                                                 ldw, bias, residual, out, ldo, M, N, K, mode, none);
        if (e != cudaSuccess) {
            mx_set_error("skinny gemm: cluster launch failed: %s", cudaGetErrorString(e));
            return (int)e;
        }
        return MX_OK;
    }
    auto kernel = M <= 8 ? gemm_skinny_kernel<1, false, false> : gemm_skinny_kernel<2, false, false>;
    if (skinny_deep(grid, K)) {
        // (both row counts: a row's sum is then formed in the same order whatever the batch)
        if (skinny_wide_ok(W, K, ldw))
            kernel = M <= 8 ? gemm_skinny_kernel<1, false, false, SK_DEEP / 2, true>
                            : gemm_skinny_kernel<2, false, false, SK_DEEP / 2, true>;
        else
            kernel = M <= 8 ? gemm_skinny_kernel<1, false, false, SK_DEEP> : gemm_skinny_kernel<2, false, false, SK_DEEP>;
    }
    mx_launch_chained(kernel, dim3(grid), dim3(SK_THREADS), 0, stream, (const __nv_bfloat16*)x, ldx,
                      (const __nv_bfloat16*)W, ldw, bias, residual, out, ldo, M, N, K, mode, none);
    return mx_launch_status();
}

// The QKV product with the rotation and the cache write in its epilogue. W is
// [(heads + 2 kv heads) * head_dim][K]; rotated queries go to `qkv` (bfloat16, row stride ldo; its
// key and value columns are left untouched), keys and values to the cache slots `slots[m]`
// (null: not stored). The rotation spans the whole head (rotary_dim == head_dim).
extern "C" int mx_gemm_skinny_rope(const void* x, const void* W, const float* bias, void* qkv, int M, int K,
                                   int ldx, int ldw, int ldo, const int* positions, const float* inv_freq,
                                   const int* slots, void* cache, long long n_pages, int n_heads,
                                   int n_kv_heads, int head_dim, int page_size, int* status,
                                   cudaStream_t stream) {
    if (M <= 0) return MX_OK;
    const int rc = check_skinny(M, K, ldx, ldw);
    if (rc != MX_OK) return rc;
    if (head_dim <= 0 || head_dim % 16 != 0) MX_REFUSE("skinny gemm with rotation: head_dim %d is no multiple of 16", head_dim);
    if (n_heads <= 0 || n_kv_heads <= 0) MX_REFUSE("skinny gemm with rotation: %d heads, %d kv heads", n_heads, n_kv_heads);
    if (slots != nullptr && cache == nullptr) MX_REFUSE("skinny gemm with rotation: slots without a cache");
    SkinnyRope rope;
    rope.positions = positions; rope.inv_freq = inv_freq; rope.slots = slots;
    rope.cache = (__nv_bfloat16*)cache; rope.status = status; rope.n_slots = n_pages * page_size;
    rope.n_heads = n_heads; rope.n_kv_heads = n_kv_heads; rope.head_dim = head_dim; rope.page_size = page_size;
    const int N = (n_heads + 2 * n_kv_heads) * head_dim;
    auto kernel = M <= 8 ? gemm_skinny_kernel<1, true, false> : gemm_skinny_kernel<2, true, false>;
    if (skinny_deep(N / 16, K)) {
        if (skinny_wide_ok(W, K, ldw))
            kernel = M <= 8 ? gemm_skinny_kernel<1, true, false, SK_DEEP / 2, true>
                            : gemm_skinny_kernel<2, true, false, SK_DEEP / 2, true>;
        else
            kernel = M <= 8 ? gemm_skinny_kernel<1, true, false, SK_DEEP> : gemm_skinny_kernel<2, true, false, SK_DEEP>;
    }
    mx_launch_chained(kernel, dim3(N / 16), dim3(SK_THREADS), 0, stream, (const __nv_bfloat16*)x, ldx,
                      (const __nv_bfloat16*)W, ldw, bias, (const float*)nullptr, qkv, ldo, M, N, K, 0, rope);
    return mx_launch_status();
}
