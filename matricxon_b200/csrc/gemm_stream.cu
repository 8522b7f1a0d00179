// out[M,N] = epilogue(x[M,K] . W[N,K]^T + bias[N]) for up to 128 rows: decoding, and prompt portions
// too short to fill prompt-sized tiles. The reference runs these products through nn.Linear
// (app/architectures/qwen_layers.py:50-53, app/architectures/starcoder2_layers.py:19-23).
//
// With so few rows the product is one pass over the weight matrix, so the kernel is a stream of W
// from HBM with the arithmetic hung on it:
//   * The roles of the operands are swapped: 128 weight rows (output features) are the M side of
//     tcgen05.mma, the tokens (padded to a multiple of 16) its N side; the accumulator
//     [feature][token] lives in tensor memory.
//   * The weight rows are dealt out evenly: with G = min(SMs, N / 8) blocks, every block owns
//     ceil(N / G) consecutive rows and walks them in tiles of at most 128 rows,
//     with all of K. One round of blocks, every SM pulls the same number of bytes, every weight byte
//     is read once by one block, and no sum is shared between blocks: a row's result depends on
//     nothing but that row (and not on the other rows of the batch).
//   * A block is six warps: warp 4 feeds a ring of stages by TMA, each stage holding a few 64-wide
//     slices of K of the block's weight rows and of the activations; warp 5 issues four
//     tcgen05.mma per slice and commits each stage back to the producer (both walk their loops as
//     whole warps with one elected lane issuing: tcgen05_helpers.cuh says why); warps 0-3 take
//     the finished accumulator out of tensor memory (a lane = a feature, a register = a token),
//     apply bias / GELU / residual on the float values and store: for one token, the 32 lanes of a
//     warp write 32 neighbouring features.
//   * A tile of fewer than 128 rows is loaded as it is (a TMA box of that many rows); the MMA still
//     reads 128 rows of shared memory (64 when the tile has at most 64: an MMA costs its read of
//     shared memory, 39 cycles for 128 rows and 23 for 64 at 16 tokens), i.e. runs on into whatever
//     follows in the ring. That only fills accumulator lanes that nobody reads: a row of the result
//     depends on its own row of W.
//   * The weights are nobody's output. Launched as a dependent of the kernel before it
//     (programmatic dependent launch), the producer fills the whole ring with weights first and only
//     then waits for that kernel to finish before it asks for activations.
// Every mbarrier wait is bounded: a wait that runs out sets MX_STATUS_WAIT_TIMEOUT and the role
// moves on, so the block always reaches the point where tensor memory is freed.
//
// Epilogue modes as in gemm_simt.cu: 0 out(bf16) = v; 1 out(bf16) = gelu_tanh(v);
// 2 out(f32) = residual + v; 3 out(f32) = v, with v = acc + bias.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05_helpers.cuh"

namespace {

constexpr int GS_THREADS = 192;            // warps 0-3 epilogue, warp 4 producer, warp 5 MMA issuer
constexpr int GS_MAX_STAGES = 12;
constexpr int GS_RING_BYTES = 176 * 1024;  // stages of weights and activations in flight per block
constexpr int GS_TAIL_BYTES = 16 * 1024;   // what a 128-row MMA may read beyond the last short tile

struct GsShared {
    unsigned long long full[GS_MAX_STAGES];
    unsigned long long empty[GS_MAX_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned tmem_base;
};

// How a product is dealt out; computed on the host, the same for every block.
struct GsPlan {
    int rows_per_block;     // consecutive weight rows a block owns
    int tile_rows;          // rows of one tile (a TMA box; at most 128)
    int tiles_per_block;
    int mpad;               // tokens padded to a multiple of 16: the N of the MMA
    int kk;                 // 64-wide slices of K per stage
    int stages;
    int groups;             // stages' worth of K per tile: ceil(ceil(K / 64) / kk)
    int tmem_cols;          // a power of two >= 32
    int mma_m;              // 128, or 64 for tiles of at most 64 rows (a shorter read of shared memory per MMA)
    unsigned w_slice_bytes, x_slice_bytes;
};

template <bool F32>
__global__ void __launch_bounds__(GS_THREADS)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                   const float* __restrict__ bias, const float* residual, void* out, int ldo, int M, int N,
                   int mode, const GsPlan plan, int* status) {
    extern __shared__ unsigned char gs_smem_raw[];
    // slices must start on a 1024-byte boundary for the 128-byte swizzle
    unsigned char* w_ring = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(gs_smem_raw) + 1023) & ~(uintptr_t)1023);
    const unsigned w_stage_bytes = (unsigned)plan.kk * plan.w_slice_bytes;
    const unsigned x_stage_bytes = (unsigned)plan.kk * plan.x_slice_bytes;
    // activations first, weights behind them: what an MMA reads beyond a short tile is then more
    // weights or the tail, never another role's data
    unsigned char* x_ring = w_ring;
    w_ring += (size_t)plan.stages * x_stage_bytes;
    __shared__ GsShared sh;

    const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
    const int row_begin = blockIdx.x * plan.rows_per_block;
    const int row_end = min(N, row_begin + plan.rows_per_block);
    const int n_tiles = (row_end - row_begin + plan.tile_rows - 1) / plan.tile_rows;

    if (threadIdx.x == 0) {
        for (int s = 0; s < plan.stages; ++s) {
            tc_mbar_init(&sh.full[s], 1);
            tc_mbar_init(&sh.empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc_mbar_init(&sh.acc_full[b], 1);
            tc_mbar_init(&sh.acc_empty[b], 4);          // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         smem_u32(&sh.tmem_base)),
                     "r"(plan.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = sh.tmem_base;

    if (warp == 4) {
        // ---------------- producer: the whole warp walks the loop, one elected lane issues (see the helpers)
        const int total = n_tiles * plan.groups;
        // what a stage's loads bring: boxes of tile_rows (not rounded) weight rows and of mpad tokens
        const unsigned stage_tx = (unsigned)plan.kk * ((unsigned)plan.tile_rows * TC_BK * 2 + plan.x_slice_bytes);
        // the ring's first filling: weights at once, activations once the kernel before this one is done
        const int ahead = min(total, plan.stages);
        for (int it = 0; it < ahead; ++it) {
            const int tile = it / plan.groups, group = it - tile * plan.groups;
            const int r0 = row_begin + tile * plan.tile_rows;
            tc_mbar_expect_tx_elect(&sh.full[it], stage_tx);
            for (int h = 0; h < plan.kk; ++h)           // columns beyond K arrive as zeros
                tma_load_2d_elect(w_ring + (size_t)it * w_stage_bytes + (size_t)h * plan.w_slice_bytes, &map_w,
                                  (group * plan.kk + h) * TC_BK, r0, &sh.full[it]);
        }
        pdl_wait();
        for (int it = 0; it < ahead; ++it) {
            const int group = it % plan.groups;
            for (int h = 0; h < plan.kk; ++h)
                tma_load_2d_elect(x_ring + (size_t)it * x_stage_bytes + (size_t)h * plan.x_slice_bytes, &map_x,
                                  (group * plan.kk + h) * TC_BK, 0, &sh.full[it]);
        }
        bool alive = true;
        for (int it = ahead; it < total && alive; ++it) {
            const int s = it % plan.stages;
            const int tile = it / plan.groups, group = it - tile * plan.groups;
            const int r0 = row_begin + tile * plan.tile_rows;
            alive = tc_mbar_wait_warp(&sh.empty[s], ((unsigned)(it / plan.stages) & 1) ^ 1, status);
            if (!alive) break;
            tc_mbar_expect_tx_elect(&sh.full[s], stage_tx);
            for (int h = 0; h < plan.kk; ++h) {
                tma_load_2d_elect(w_ring + (size_t)s * w_stage_bytes + (size_t)h * plan.w_slice_bytes, &map_w,
                                  (group * plan.kk + h) * TC_BK, r0, &sh.full[s]);
                tma_load_2d_elect(x_ring + (size_t)s * x_stage_bytes + (size_t)h * plan.x_slice_bytes, &map_x,
                                  (group * plan.kk + h) * TC_BK, 0, &sh.full[s]);
            }
        }
        // everything this block will ever ask for is on its way: the next kernel may begin its own
        // preamble (its weights) on the SMs that free up
        pdl_trigger();
        // no copy of this block may still be in flight when it ends: wait (bounded) for the
        // loads of the last stages to land
        for (int j = max(0, total - plan.stages); j < total; ++j)
            if (!tc_mbar_wait_warp(&sh.full[j % plan.stages], (unsigned)(j / plan.stages) & 1, status)) break;
    } else if (warp == 5) {
        // ---------------- MMA issuer: the whole warp walks the loop, one elected lane issues
        const unsigned idesc = umma_idesc(plan.mma_m, plan.mpad);
        int it = 0;
        bool alive = true;
        for (int tile = 0; tile < n_tiles && alive; ++tile) {
            const int buf = tile & 1;
            alive = tc_mbar_wait_warp(&sh.acc_empty[buf], ((unsigned)(tile >> 1) & 1) ^ 1, status);
            if (!alive) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned tmem_acc = tmem_base + (unsigned)(buf * plan.mpad);
            for (int group = 0; group < plan.groups; ++group, ++it) {
                const int s = it % plan.stages;
                alive = tc_mbar_wait_warp(&sh.full[s], (unsigned)(it / plan.stages) & 1, status);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                unsigned long long adesc = umma_desc(w_ring + (size_t)s * w_stage_bytes);
                unsigned long long bdesc = umma_desc(x_ring + (size_t)s * x_stage_bytes);
                for (int h = 0; h < plan.kk; ++h) {
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)   // 16 elements = 32 bytes further along K
                        umma_bf16_elect(tmem_acc, adesc + 2 * k, bdesc + 2 * k, idesc, (group | h | k) != 0);
                    adesc += plan.w_slice_bytes >> 4;
                    bdesc += plan.x_slice_bytes >> 4;
                }
                umma_commit_elect(&sh.empty[s]);
            }
            if (alive) umma_commit_elect(&sh.acc_full[buf]);   // arrives when the tile's MMAs are done
        }
    } else {
        // ---------------- epilogue: warp w owns accumulator lanes (features) 32 w .. 32 w + 31
        pdl_wait();                                          // the residual is somebody's output
        for (int tile = 0; tile < n_tiles; ++tile) {
            const int buf = tile & 1;
            const int r0 = row_begin + tile * plan.tile_rows;
            // an accumulator of 128 rows has row r in lane r; one of 64 rows has row r in lane
            // 32 (r / 16) + r % 16, i.e. every warp's first 16 lanes hold 16 rows
            const int in_tile = plan.mma_m == 128 ? 32 * warp + lane : (lane < 16 ? 16 * warp + lane : plan.tile_rows);
            const int n = r0 + in_tile;
            const bool live = in_tile < plan.tile_rows && n < row_end;
            const float b = (live && bias != nullptr) ? bias[n] : 0.f;
            if (!tc_mbar_wait(&sh.acc_full[buf], (unsigned)(tile >> 1) & 1, status)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned tbase = tmem_base + (unsigned)(buf * plan.mpad) + ((unsigned)(32 * warp) << 16);
            if ((plan.mma_m == 128 ? 32 : 16) * warp < plan.tile_rows) {
                for (int c0 = 0; c0 < plan.mpad; c0 += 16) {
                    unsigned r[16];
                    tmem_load16(tbase + (unsigned)c0, r);
                    if (!live) continue;
                    if constexpr (F32) {
                        // the residual values of the piece set out together, before any of them is needed
                        // (an element is read and written by this thread alone, also when the sum goes
                        // back in place)
                        float res[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            res[j] = (mode == 2 && c0 + j < M) ? __ldcg(residual + (size_t)(c0 + j) * ldo + n) : 0.f;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < M)
                                reinterpret_cast<float*>(out)[(size_t)(c0 + j) * ldo + n] = __uint_as_float(r[j]) + b + res[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (c0 + j >= M) break;
                            float v = __uint_as_float(r[j]) + b;
                            if (mode == 1) v = gelu_tanh_fast(v);
                            reinterpret_cast<__nv_bfloat16*>(out)[(size_t)(c0 + j) * ldo + n] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
            // the accumulator buffer may be overwritten from here on
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&sh.acc_empty[buf]);
        }
    }
    // ---------------- teardown: every role arrives here; then tensor memory is freed
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 5) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base),
                     "r"(plan.tmem_cols)
                     : "memory");
    }
}

int gs_sm_count() {
    static int count = 0;
    if (count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
        if (count <= 0) count = 148;
    }
    return count;
}

int gs_round_up(int v, int to) { return (v + to - 1) / to * to; }

}  // namespace

extern "C" int mx_gemm_stream(const void* x, const void* W, const float* bias, const float* residual, void* out,
                              int out_dtype, int M, int N, int K, int ldx, int ldw, int ldo, int mode,
                              int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return MX_OK;
    if (M > 128) MX_REFUSE("streaming gemm: %d rows, this kernel takes at most 128", M);
    if (K <= 0 || K % 8 != 0) MX_REFUSE("streaming gemm: K = %d is not a positive multiple of 8", K);
    if (ldx % 8 != 0 || ldw % 8 != 0) MX_REFUSE("streaming gemm: row strides %d, %d are not multiples of 8", ldx, ldw);
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W)) & 15)
        MX_REFUSE("streaming gemm: operands must start on 16-byte boundaries");
    if (mode < 0 || mode > 3) MX_REFUSE("streaming gemm: unknown epilogue mode %d", mode);
    if (mode == 2 && residual == nullptr) MX_REFUSE("streaming gemm: residual mode without a residual");
    if ((mode >= 2) != (out_dtype == MX_DTYPE_F32))
        MX_REFUSE("streaming gemm: epilogue mode %d does not write dtype %d", mode, out_dtype);
    if (status == nullptr) MX_REFUSE("streaming gemm: a status word is needed for its bounded waits");

    GsPlan plan;
    const int n_sm = gs_sm_count();
    const int blocks_wanted = min(n_sm, (N + 7) / 8);
    plan.rows_per_block = (N + blocks_wanted - 1) / blocks_wanted;
    const int grid = (N + plan.rows_per_block - 1) / plan.rows_per_block;
    plan.tiles_per_block = (plan.rows_per_block + 127) / 128;
    plan.tile_rows = (plan.rows_per_block + plan.tiles_per_block - 1) / plan.tiles_per_block;
    plan.mpad = gs_round_up(M, 16);
    plan.mma_m = plan.tile_rows <= 64 ? 64 : 128;
    // a slice of a tile in shared memory: whole groups of eight rows (the swizzle's unit, 1024 bytes)
    plan.w_slice_bytes = (unsigned)gs_round_up(plan.tile_rows, 8) * TC_BK * 2;
    plan.x_slice_bytes = (unsigned)plan.mpad * TC_BK * 2;
    const int slice = (int)(plan.w_slice_bytes + plan.x_slice_bytes);
    const int k_slices = (K + TC_BK - 1) / TC_BK;
    // stages of about 32 KB: the cost of a stage (a barrier round trip for the producer and for the
    // issuer) is then small beside its bytes, and enough stages fit for the ring to cover the latency
    plan.kk = max(1, min(min(8, k_slices), (32 * 1024) / slice));
    plan.stages = max(2, min(GS_MAX_STAGES, GS_RING_BYTES / (plan.kk * slice)));
    plan.groups = (k_slices + plan.kk - 1) / plan.kk;
    const int acc_cols = plan.tiles_per_block > 1 ? 2 * plan.mpad : plan.mpad;
    plan.tmem_cols = 32;
    while (plan.tmem_cols < acc_cols) plan.tmem_cols *= 2;

    CUtensorMap map_x, map_w;
    int rc = mx_tensor_map_2d(&map_x, x, M, K, ldx, plan.mpad);
    if (rc != MX_OK) return rc;
    rc = mx_tensor_map_2d(&map_w, W, N, K, ldw, plan.tile_rows);
    if (rc != MX_OK) return rc;
    const size_t smem = (size_t)plan.stages * plan.kk * slice + GS_TAIL_BYTES + 1024;
    static bool attribute_set = false;
    if (!attribute_set) {
        const int most = 226 * 1024;
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) MX_REFUSE("streaming gemm: cannot reserve %d bytes of shared memory", most);
        attribute_set = true;
    }
    cudaError_t e;
    if (out_dtype == MX_DTYPE_F32)
        e = mx_launch_chained(gemm_stream_kernel<true>, dim3(grid), dim3(GS_THREADS), smem, stream, map_x, map_w, bias,
                              residual, out, ldo, M, N, mode, plan, status);
    else
        e = mx_launch_chained(gemm_stream_kernel<false>, dim3(grid), dim3(GS_THREADS), smem, stream, map_x, map_w, bias,
                              residual, out, ldo, M, N, mode, plan, status);
    if (e != cudaSuccess) {
        mx_set_error("streaming gemm: launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return MX_OK;
}
