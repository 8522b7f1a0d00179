// out[M,N] = epilogue(A[M,K] . W[N,K]^T + bias[N]) on the 5th-generation tensor cores.
//
// bfloat16 operands, float accumulation in tensor memory, bias / GELU / residual applied to
// the float accumulator before the one rounding: the product behind every Linear of the
// reference (app/architectures/qwen_layers.py:50-53, app/architectures/starcoder2_layers.py:19-23)
// for prompt-sized M, with no separate epilogue pass over the activations.
//
// A block walks 128 x BN tiles of the output (BN a multiple of 16 up to 256, chosen per shape so
// that the SMs get even shares) in six warps:
//   warp 4, one lane: producer. For every 64-wide slice of K it waits for a free stage,
//     announces the bytes on the stage's "full" mbarrier and issues two TMA tile loads
//     (cp.async.bulk.tensor.2d, 128-byte swizzle) for A and W, both K-major.
//   warp 5, one lane: MMA issuer. Waits for "full", issues four tcgen05.mma (K = 16 each) whose
//     operands are shared-memory descriptors over the swizzled stage, and commits them to the
//     stage's "empty" mbarrier; after the last slice it commits to the "accumulator ready"
//     mbarrier of the accumulator buffer in use. Warp 5 also allocates and frees tensor memory
//     (all 512 columns: two accumulator buffers, so one block per SM).
//   warps 0-3: epilogue. Each owns 32 of the 128 accumulator lanes (rows): tcgen05.ld brings
//     32 columns at a time into registers; the piece crosses a swizzled 4 KB stage in shared memory
//     so that eight lanes carry one row piece out together, and bias / GELU / residual are applied
//     on the way (EpilogueLane below). Outputs whose rows are not 16-byte aligned take the plain
//     way: every lane stores its own row 16 columns at a time.
// Rows and columns beyond M, N and K are zero-filled by TMA on the way in and skipped on the
// way out. Every mbarrier wait is bounded: a wait that runs out sets MX_STATUS_WAIT_TIMEOUT in
// the status word and the role moves on, so the block always reaches the point where tensor
// memory is freed.
//
// Three kernels share this scheme: 128-row tiles (below), 256-row tiles (two accumulators per block) and
// 512-row tiles on pairs of SMs (cta_group::2); mx_gemm_tcgen05 picks by the number of rows.
//
// Epilogue modes as in gemm_simt.cu: 0 out(bf16) = v; 1 out(bf16) = gelu_tanh(v);
// 2 out(f32) = residual + v; 3 out(f32) = v, with v = acc + bias.
#include <cuda.h>

#include <cstdlib>

#include <mutex>

#include "common.cuh"
#include "tcgen05_helpers.cuh"

namespace {

constexpr int TC_BM = 128;
constexpr int TC_STAGES = 4;
constexpr int TC_THREADS = 192;
constexpr int TC_STAGING = 4 * 4096;      // a 4 KB stage for each epilogue warp

struct TcShared {
    unsigned long long full[TC_STAGES];
    unsigned long long empty[TC_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned tmem_base;
};

// Applies the epilogue to 16 accumulator values of one output row and stores them.
__device__ __forceinline__ void store_piece(const unsigned (&r)[16], const float* __restrict__ bias,
                                            const float* residual, void* out, size_t obase, int nbase, int N,
                                            int mode) {
    if (mode >= 2) {
        float* o = reinterpret_cast<float*>(out) + obase;
        const float* res = (mode == 2) ? residual + obase : nullptr;
        if (nbase + 16 <= N && (obase % 4) == 0) {
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
                float4 v;
                v.x = __uint_as_float(r[j]); v.y = __uint_as_float(r[j + 1]);
                v.z = __uint_as_float(r[j + 2]); v.w = __uint_as_float(r[j + 3]);
                if (bias) {
                    v.x += bias[nbase + j]; v.y += bias[nbase + j + 1];
                    v.z += bias[nbase + j + 2]; v.w += bias[nbase + j + 3];
                }
                if (res) {
                    const float4 q = *reinterpret_cast<const float4*>(res + j);
                    v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
                }
                *reinterpret_cast<float4*>(o + j) = v;
            }
        } else {
            for (int j = 0; j < 16; ++j) {
                if (nbase + j >= N) break;
                float v = __uint_as_float(r[j]);
                if (bias) v += bias[nbase + j];
                if (res) v += res[j];
                o[j] = v;
            }
        }
        return;
    }
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + obase;
    if (nbase + 16 <= N && (obase % 8) == 0) {
#pragma unroll
        for (int j = 0; j < 16; j += 8) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[e] = __uint_as_float(r[j + e]);
                if (bias) v[e] += bias[nbase + j + e];
                if (mode == 1) v[e] = gelu_tanh_fast(v[e]);
            }
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(v[2], v[3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(v[6], v[7]);
            pk.x = *reinterpret_cast<unsigned*>(&h0); pk.y = *reinterpret_cast<unsigned*>(&h1);
            pk.z = *reinterpret_cast<unsigned*>(&h2); pk.w = *reinterpret_cast<unsigned*>(&h3);
            *reinterpret_cast<uint4*>(o + j) = pk;
        }
    } else {
        for (int j = 0; j < 16; ++j) {
            if (nbase + j >= N) break;
            float v = __uint_as_float(r[j]);
            if (bias) v += bias[nbase + j];
            if (mode == 1) v = gelu_tanh_fast(v);
            o[j] = __float2bfloat16_rn(v);
        }
    }
}

// Epilogue warps per 32 accumulator lanes and accumulator (they take 32-column pieces in turn): one.
constexpr int TCP_PARTS = 1;

__device__ __forceinline__ void mbar_arrive_cluster(unsigned bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ void tmem_load32_nowait(unsigned taddr, unsigned* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// Shared-memory accesses by 32-bit shared address: the stage pointers are computed through integers, so the
// compiler would otherwise use generic loads and stores (slower, and ordered against the global ones).
__device__ __forceinline__ void sts128(unsigned addr, unsigned a, unsigned b, unsigned c, unsigned d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ float4 lds128(unsigned addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

// out[0..3] += v without reading it here: the addition happens at the memory side, nothing waits for it.
__device__ __forceinline__ void red_add_f32x4(float* dst, float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

// A warp's 32 rows of one accumulator leave through shared memory so that global memory sees whole
// row pieces: 32 columns at a time, every lane writes its own row's 32 floats into the warp's stage
// in a 16-byte XOR swizzle; then eight lanes together carry one row piece out (four rows per
// instruction), and that is where bias, residual, GELU and the rounding are applied: a lane keeps one
// 4-column unit for all rows. The loop hardly waits on global memory: the bias unit of a piece is
// fetched one piece ahead (the first by `EpilogueLane::prefetch` while the products still run), the
// residual pieces set out together with the accumulator piece they belong to, and for bfloat16
// outputs the next accumulator piece is on its way from tensor memory while one is carried out. No bank conflicts either way. `stage`: 4 KB of this warp.
// `free_bar`: arrived on by lane 0 as soon as the warp has read its last accumulator value.
template <bool F32>
struct EpilogueLane {
    float4 bias4;             // this lane's bias unit of the coming 32-column piece
    float4 res[8];            // residual pieces of the coming 32-column piece (rows 4 i + lane / 8)
    int sub_row, unit_out;

    __device__ __forceinline__ void load_bias(const float* __restrict__ bias, int n0, int c, int bn, int N) {
        const int col_out = n0 + c + unit_out * 4;
        bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias != nullptr && c + unit_out * 4 < bn && col_out < N) {
            if (col_out + 4 <= N) bias4 = __ldg(reinterpret_cast<const float4*>(bias + col_out));
            else {
                bias4.x = bias[col_out];
                if (col_out + 1 < N) bias4.y = bias[col_out + 1];
                if (col_out + 2 < N) bias4.z = bias[col_out + 2];
            }
        }
    }

    __device__ __forceinline__ void load_residual(const float* residual, int ldo, int row0, int n0, int c,
                                                  int bn, int M, int N) {
        const int col_out = n0 + c + unit_out * 4;
        const bool live = c < bn && unit_out * 4 < bn - c && col_out < N;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int row = row0 + 4 * i + sub_row;
            res[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live && row < M) {
                const float* src = residual + (size_t)row * ldo + col_out;
                if (col_out + 4 <= N) res[i] = *reinterpret_cast<const float4*>(src);
                else {
                    res[i].x = src[0];
                    if (col_out + 1 < N) res[i].y = src[1];
                    if (col_out + 2 < N) res[i].z = src[2];
                }
            }
        }
    }

    // Before the accumulator is waited for: what the first piece needs from global memory.
    __device__ __forceinline__ void prefetch(const float* __restrict__ bias, const float* residual,
                                             const void* out, int ldo, int row0, int n0, int c_first, int bn,
                                             int M, int N, int mode, int lane) {
        sub_row = lane >> 3;
        unit_out = lane & 7;
        load_bias(bias, n0, c_first, bn, N);
        if constexpr (F32) {
            if (mode == 2 && residual != out) load_residual(residual, ldo, row0, n0, c_first, bn, M, N);
        }
    }

    // One 32-column piece: `cur` holds (after the wait) the accumulator values of columns c .. c + 31 of
    // this lane's row; the next piece is sent for into `nxt`.
    __device__ __forceinline__ void piece(unsigned* cur, unsigned* nxt, int c, unsigned tbase, int row0, int n0,
                                          int bn, const float* __restrict__ bias, const float* residual,
                                          void* out, int ldo, int M, int N, int mode, unsigned char* stage,
                                          int lane, unsigned free_bar) {
        const int c_next = c + 32 * TCP_PARTS;
        const bool last = c_next >= bn;
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        const float4 b4 = bias4;
        if (!last) load_bias(bias, n0, c_next, bn, N);
        if constexpr (!F32) {
            if (!last) tmem_load32_nowait(tbase + (unsigned)c_next, nxt);
        }
        if (last) {                                      // the accumulator may be overwritten from here on
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(free_bar);
        }
        if (row0 < M && n0 + c < N) {
            const unsigned stage_addr = smem_u32(stage);
            const unsigned row_dst = stage_addr + lane * 128;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                sts128(row_dst + ((u ^ (lane & 7)) << 4), cur[4 * u], cur[4 * u + 1], cur[4 * u + 2], cur[4 * u + 3]);
            __syncwarp();
            if (row0 + 32 <= M && n0 + c + 32 <= N && c + 32 <= bn) {
                // every row and column of the piece exists: no predicates, vector accesses only
                float4 v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int local_row = 4 * i + sub_row;
                    v[i] = lds128(stage_addr + local_row * 128 + ((unit_out ^ (local_row & 7)) << 4));
                }
                const size_t first = (size_t)(row0 + sub_row) * ldo + n0 + c + unit_out * 4;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v[i].x += b4.x; v[i].y += b4.y; v[i].z += b4.z; v[i].w += b4.w;
                    if constexpr (F32) {
                        float* dst = reinterpret_cast<float*>(out) + first + (size_t)(4 * i) * ldo;
                        if (mode == 2 && residual == out) {
                            red_add_f32x4(dst, v[i]);    // the residual stream is updated in place
                        } else {
                            if (mode == 2) {
                                v[i].x += res[i].x; v[i].y += res[i].y; v[i].z += res[i].z; v[i].w += res[i].w;
                            }
                            *reinterpret_cast<float4*>(dst) = v[i];
                        }
                    } else {
                        if (mode == 1) {
                            v[i].x = gelu_tanh_fast(v[i].x); v[i].y = gelu_tanh_fast(v[i].y);
                            v[i].z = gelu_tanh_fast(v[i].z); v[i].w = gelu_tanh_fast(v[i].w);
                        }
                        __nv_bfloat162 lo = __floats2bfloat162_rn(v[i].x, v[i].y);
                        __nv_bfloat162 hi = __floats2bfloat162_rn(v[i].z, v[i].w);
                        uint2 pk;
                        pk.x = *reinterpret_cast<unsigned*>(&lo); pk.y = *reinterpret_cast<unsigned*>(&hi);
                        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + first +
                                                  (size_t)(4 * i) * ldo) = pk;
                    }
                }
            } else {
                edge_piece(stage_addr, c, row0, n0, bn, b4, residual, out, ldo, M, N, mode);
            }
            __syncwarp();                                // the stage is free for the next piece
        }
        if constexpr (F32) {                             // the next piece and its residual set out together
            if (!last) {
                tmem_load32_nowait(tbase + (unsigned)c_next, nxt);
                if (mode == 2 && residual != out) load_residual(residual, ldo, row0, n0, c_next, bn, M, N);
            }
        }
    }

    // The same way out for a piece that crosses the last row, the last column or the tile's width: every
    // access is checked. Kept out of line so that the loop over interior pieces stays short.
    __device__ __noinline__ void edge_piece(unsigned stage_addr, int c, int row0, int n0, int bn, float4 b4,
                                            const float* residual, void* out, int ldo, int M, int N, int mode) {
        const int width = min(32, bn - c);
        const int col_out = n0 + c + unit_out * 4;
        if (unit_out * 4 >= width || col_out >= N) return;
        for (int i = 0; i < 8; ++i) {
            const int local_row = 4 * i + sub_row, row = row0 + local_row;
            if (row >= M) continue;
            const float4 staged = lds128(stage_addr + local_row * 128 + ((unit_out ^ (local_row & 7)) << 4));
            float v[4] = {staged.x + b4.x, staged.y + b4.y, staged.z + b4.z, staged.w + b4.w};
            for (int e = 0; e < 4 && col_out + e < N; ++e) {
                const size_t at = (size_t)row * ldo + col_out + e;
                if constexpr (F32) {
                    float* dst = reinterpret_cast<float*>(out) + at;
                    if (mode == 2 && residual == out) atomicAdd(dst, v[e]);
                    else *dst = (mode == 2 ? residual[at] : 0.f) + v[e];
                } else {
                    reinterpret_cast<__nv_bfloat16*>(out)[at] =
                        __float2bfloat16_rn(mode == 1 ? gelu_tanh_fast(v[e]) : v[e]);
                }
            }
        }
    }

    // The loops over pieces stay rolled: code that runs once per tile is fetched cold, and a block
    // spends longer waiting for the instructions of an unrolled epilogue than executing them.
    __device__ __forceinline__ void drain(unsigned tbase, int row0, int n0, int c_first, int bn,
                                          const float* __restrict__ bias, const float* residual, void* out,
                                          int ldo, int M, int N, int mode, unsigned char* stage, int lane,
                                          unsigned free_bar) {
        constexpr int STEP = 32 * TCP_PARTS;
        if (c_first >= bn) {                             // a tile too narrow to give this warp a piece
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(free_bar);
            return;
        }
        unsigned ra[32];
        tmem_load32_nowait(tbase + (unsigned)c_first, ra);
        if constexpr (F32) {                             // one register buffer: the others hold the residual
#pragma unroll 1
            for (int c = c_first; c < bn; c += STEP)
                piece(ra, ra, c, tbase, row0, n0, bn, bias, residual, out, ldo, M, N, mode, stage, lane, free_bar);
        } else {
            unsigned rb[32];
#pragma unroll 1
            for (int c = c_first; c < bn; c += 2 * STEP) {
                piece(ra, rb, c, tbase, row0, n0, bn, bias, residual, out, ldo, M, N, mode, stage, lane, free_bar);
                if (c + STEP < bn)
                    piece(rb, ra, c + STEP, tbase, row0, n0, bn, bias, residual, out, ldo, M, N, mode, stage, lane,
                          free_bar);
            }
        }
    }
};


// Persistent: a block walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ... (rows fastest, so
// blocks that run together share weight tiles through L2). The accumulator is double-buffered
// in tensor memory (2 x 256 columns): the epilogue of one tile overlaps the products of the next.
// `staged`: the epilogue goes through the 4 KB stages behind the operand stages (coalesced stores; needs
// 16-byte-aligned rows, see mx_gemm_tcgen05); otherwise every lane stores its own row's pieces.
template <bool F32>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, const float* residual, void* out, int ldo, int M,
                    int N, int K, int bn, int mode, int staged, int kk, int* status) {
    const unsigned a_bytes = TC_BM * TC_BK * 2, w_bytes = (unsigned)bn * TC_BK * 2;
    // kk slices of K (64 wide each) share a stage and its barrier: with narrow tiles the fixed cost of a
    // stage (a barrier round trip in the producer and in the issuer) is what bounds the main loop
    const unsigned stage_bytes = (unsigned)kk * (a_bytes + w_bytes);
    extern __shared__ unsigned char tc_smem_raw[];
    // stages must start on a 1024-byte boundary for the 128-byte swizzle
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ TcShared sh;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_slices = ((K + TC_BK - 1) / TC_BK + kk - 1) / kk;          // in stages
    const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (N + bn - 1) / bn;
    const int n_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
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
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = sh.tmem_base;

    if (warp == 4) {
        // ---------------- producer
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * bn;
                for (int ks = 0; ks < k_slices; ++ks, ++it) {
                    const int s = it % TC_STAGES;
                    alive = tc_mbar_wait(&sh.empty[s], ((unsigned)(it / TC_STAGES) & 1) ^ 1, status);
                    if (!alive) break;
                    tc_mbar_expect_tx(&sh.full[s], stage_bytes);
                    unsigned char* a_tile = tiles + (size_t)s * stage_bytes;
                    for (int h = 0; h < kk; ++h) {          // columns beyond K arrive as zeros
                        tma_load_2d(a_tile + h * a_bytes, &map_a, (ks * kk + h) * TC_BK, m0, &sh.full[s]);
                        tma_load_2d(a_tile + kk * a_bytes + h * w_bytes, &map_w, (ks * kk + h) * TC_BK, n0,
                                    &sh.full[s]);
                    }
                }
            }
            // no copy of this block may still be in flight when it ends: wait (bounded) for the
            // loads of the last stages to land
            for (int j = max(0, it - TC_STAGES); j < it; ++j)
                if (!tc_mbar_wait(&sh.full[j % TC_STAGES], (unsigned)(j / TC_STAGES) & 1, status)) break;
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer
        if (lane == 0) {
            const unsigned idesc = umma_idesc(TC_BM, bn);
            int it = 0, local = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                alive = tc_mbar_wait(&sh.acc_empty[buf], ((unsigned)(local >> 1) & 1) ^ 1, status);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned tmem_acc = tmem_base + (unsigned)buf * 256;
                for (int ks = 0; ks < k_slices; ++ks, ++it) {
                    const int s = it % TC_STAGES;
                    alive = tc_mbar_wait(&sh.full[s], (unsigned)(it / TC_STAGES) & 1, status);
                    if (!alive) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned char* a_tile = tiles + (size_t)s * stage_bytes;
                    for (int h = 0; h < kk; ++h) {
                        const unsigned long long adesc = umma_desc(a_tile + h * a_bytes);
                        const unsigned long long bdesc = umma_desc(a_tile + kk * a_bytes + h * w_bytes);
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; ++k)   // 16 elements = 32 bytes further along K
                            umma_bf16(tmem_acc, adesc + 2 * k, bdesc + 2 * k, idesc, (ks | h | k) != 0);
                    }
                    umma_commit(&sh.empty[s]);
                }
                if (alive) umma_commit(&sh.acc_full[buf]);   // arrives when the tile's MMAs are done
            }
        }
    } else {
        // ---------------- epilogue: warp w owns accumulator lanes 32 w .. 32 w + 31
        int local = 0;
        unsigned char* stage = tiles + (size_t)TC_STAGES * stage_bytes + (size_t)warp * 4096;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * bn;
            const unsigned tbase = tmem_base + (unsigned)buf * 256 + ((unsigned)(32 * warp) << 16);
            if (staged) {
                EpilogueLane<F32> mine;
                mine.prefetch(bias, residual, out, ldo, m0 + 32 * warp, n0, 0, bn, M, N, mode, lane);
                if (!tc_mbar_wait(&sh.acc_full[buf], (unsigned)(local >> 1) & 1, status)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                mine.drain(tbase, m0 + 32 * warp, n0, 0, bn, bias, residual, out, ldo, M, N, mode, stage, lane,
                           smem_u32(&sh.acc_empty[buf]));
                continue;
            }
            if (!tc_mbar_wait(&sh.acc_full[buf], (unsigned)(local >> 1) & 1, status)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int row = m0 + 32 * warp + lane;
            for (int c0 = 0; c0 < bn; c0 += 16) {
                unsigned r[16];
                tmem_load16(tbase + (unsigned)c0, r);
                if (row < M && n0 + c0 < N)
                    store_piece(r, bias, residual, out, (size_t)row * ldo + n0 + c0, n0 + c0, N, mode);
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The same product with 256-row tiles (and, for a residual added in place, K shared out between
// blocks: with few rows a product has too few tiles for 148 SMs, and what bounds a block is what it
// loads): two 128 x BN accumulators share every weight tile, so a
// block takes in (256 + BN) x 128 bytes per 64-wide slice of K for twice the arithmetic. What a
// block can keep in flight (its shared memory) divided by the latency of a TMA load is its
// bandwidth; with 128-row tiles that bandwidth feeds the tensor pipe for about 40 % of the
// time, with 256-row tiles for most of it. The two accumulators fill tensor memory (2 x 256
// columns), so the epilogue of a tile does not overlap the next tile's products; eight
// epilogue warps (two per lane quarter, one per accumulator) keep it short, and the producer
// goes on loading the next tile's stages meanwhile.
constexpr int TCW_BM = 256;
constexpr int TCW_STAGES = 3;
constexpr int TCW_THREADS = 320;      // warps 0-7 epilogue, warp 8 producer, warp 9 MMA issuer
constexpr int TCW_STAGING = 8 * 4096;  // a 4 KB stage for each epilogue warp

struct TcWideShared {
    unsigned long long full[TCW_STAGES];
    unsigned long long empty[TCW_STAGES];
    unsigned long long acc_full;
    unsigned long long acc_empty;
    unsigned tmem_base;
};


template <bool F32>
__global__ void __launch_bounds__(TCW_THREADS)
gemm_tcgen05_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const float* __restrict__ bias, const float* residual, void* out, int ldo, int M,
                         int N, int K, int bn, int mode, int k_splits, int* status) {
    const unsigned a_bytes = TCW_BM * TC_BK * 2, w_bytes = (unsigned)bn * TC_BK * 2;
    const unsigned stage_bytes = a_bytes + w_bytes;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ TcWideShared sh;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_slices = (K + TC_BK - 1) / TC_BK;
    const int tiles_m = (M + TCW_BM - 1) / TCW_BM, tiles_n = (N + bn - 1) / bn;
    const int n_tiles = tiles_m * tiles_n;
    // k_splits > 1: a tile's slices of K are shared out between that many work items, each of which adds
    // its part into the output (residual mode in place only: the additions happen at the memory side)
    const int per_split = (k_slices + k_splits - 1) / k_splits;
    const int n_items = n_tiles * k_splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TCW_STAGES; ++s) {
            tc_mbar_init(&sh.full[s], 1);
            tc_mbar_init(&sh.empty[s], 1);
        }
        tc_mbar_init(&sh.acc_full, 1);
        tc_mbar_init(&sh.acc_empty, 8);                 // one arrival per epilogue warp
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         smem_u32(&sh.tmem_base)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = sh.tmem_base;

    if (warp == 8) {
        // ---------------- producer
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
                const int tile = item / k_splits, split = item - tile * k_splits;
                const int m0 = (tile % tiles_m) * TCW_BM, n0 = (tile / tiles_m) * bn;
                const int ks_end = min(k_slices, (split + 1) * per_split);
                for (int ks = split * per_split; ks < ks_end; ++ks, ++it) {
                    const int s = it % TCW_STAGES;
                    alive = tc_mbar_wait(&sh.empty[s], ((unsigned)(it / TCW_STAGES) & 1) ^ 1, status);
                    if (!alive) break;
                    tc_mbar_expect_tx(&sh.full[s], stage_bytes);
                    unsigned char* a_tile = tiles + (size_t)s * stage_bytes;
                    tma_load_2d(a_tile, &map_a, ks * TC_BK, m0, &sh.full[s]);
                    tma_load_2d(a_tile + a_bytes, &map_w, ks * TC_BK, n0, &sh.full[s]);
                }
            }
            for (int j = max(0, it - TCW_STAGES); j < it; ++j)     // nothing of ours stays in flight
                if (!tc_mbar_wait(&sh.full[j % TCW_STAGES], (unsigned)(j / TCW_STAGES) & 1, status)) break;
        }
    } else if (warp == 9) {
        // ---------------- MMA issuer: rows 0-127 into columns [0, bn), rows 128-255 into [256, 256 + bn)
        if (lane == 0) {
            const unsigned idesc = umma_idesc(128, bn);
            int it = 0, local = 0;
            bool alive = true;
            for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x, ++local) {
                const int split = item % k_splits;
                const int ks_begin = split * per_split, ks_end = min(k_slices, ks_begin + per_split);
                alive = tc_mbar_wait(&sh.acc_empty, ((unsigned)local & 1) ^ 1, status);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                for (int ks = ks_begin; ks < ks_end; ++ks, ++it) {
                    const int s = it % TCW_STAGES;
                    alive = tc_mbar_wait(&sh.full[s], (unsigned)(it / TCW_STAGES) & 1, status);
                    if (!alive) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned char* a_tile = tiles + (size_t)s * stage_bytes;
                    const unsigned long long adesc_lo = umma_desc(a_tile);
                    const unsigned long long adesc_hi = umma_desc(a_tile + 128 * TC_BK * 2);
                    const unsigned long long bdesc = umma_desc(a_tile + a_bytes);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {
                        umma_bf16(tmem_base, adesc_lo + 2 * k, bdesc + 2 * k, idesc, ks > ks_begin || k != 0);
                        umma_bf16(tmem_base + 256, adesc_hi + 2 * k, bdesc + 2 * k, idesc, ks > ks_begin || k != 0);
                    }
                    umma_commit(&sh.empty[s]);
                }
                if (alive) umma_commit(&sh.acc_full);
            }
        }
    } else {
        // ---------------- epilogue: warp w -> accumulator w / 4, lane quarter w % 4
        const int half = warp >> 2, quarter = warp & 3;
        const unsigned free_bar = smem_u32(&sh.acc_empty);
        unsigned char* stage = tiles + (size_t)TCW_STAGES * stage_bytes + (size_t)warp * 4096;
        int local = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++local) {
            const int tile = item / k_splits, split = item - tile * k_splits;
            const int m0 = (tile % tiles_m) * TCW_BM, n0 = (tile / tiles_m) * bn;
            const int row0 = m0 + 128 * half + 32 * quarter;
            const unsigned tbase = tmem_base + (unsigned)half * 256 + ((unsigned)(32 * quarter) << 16);
            const float* bias_here = split == 0 ? bias : nullptr;     // one of a tile's parts brings the bias
            EpilogueLane<F32> mine;
            mine.prefetch(bias_here, residual, out, ldo, row0, n0, 0, bn, M, N, mode, lane);
            if (!tc_mbar_wait(&sh.acc_full, (unsigned)local & 1, status)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            mine.drain(tbase, row0, n0, 0, bn, bias_here, residual, out, ldo, M, N, mode, stage, lane, free_bar);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 9) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The same product on pairs of SMs (tcgen05 cta_group::2): a cluster of two blocks works on one
// 512 x BN tile. Every MMA spans both SMs (M = 256: rows 0-127 accumulate in the first block's tensor
// memory, rows 128-255 in the second's) and reads its B operand half from each block's shared
// memory, so a block takes in 256 rows of A and only BN / 2 rows of W per slice of K: 48 KB where
// the 256-row kernel needs 64 KB for the same arithmetic, and four stages fit where it has three.
// That is what this product is bound by: bytes in flight per SM over the latency of a load.
//   Both blocks run a producer (warp 8): it waits for its own "empty" barrier and issues its loads,
//   which all announce their bytes on the FIRST block's "full" barrier (the cta_group::2 form of
//   the TMA load may signal the peer's barrier). The first block's warp 9 issues the MMAs for the
//   pair and commits them to the "empty" / "accumulator ready" barriers of both blocks (commit with
//   a block mask). Warps 0-7 of each block drain that block's 128 lanes of both accumulators and
//   arrive on the first block's "accumulator free" barrier (16 arrivals).
// No load here is a multicast: each block fetches what it holds.
constexpr int TCP_ROWS = 512;          // rows of a pair's tile
constexpr int TCP_EPI_WARPS = 8 * TCP_PARTS;
constexpr int TCP_STAGES = TCP_PARTS == 1 ? 4 : 3;
constexpr int TCP_THREADS = 32 * (TCP_EPI_WARPS + 2);    // then the producer warp and the MMA warp
constexpr int TCP_STAGING = TCP_EPI_WARPS * 4096;        // a 4 KB stage for each epilogue warp

struct TcPairShared {
    unsigned long long full[TCP_STAGES];       // used in the first block of the pair
    unsigned long long empty[TCP_STAGES];      // in each block
    unsigned long long acc_full;               // in each block
    unsigned long long acc_empty;              // used in the first block: 16 arrivals
    unsigned tmem_base;
};

__device__ __forceinline__ unsigned cluster_block_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// The address of the same shared-memory object in block `rank` of the cluster.
__device__ __forceinline__ unsigned shared_of_rank(const void* ptr, unsigned rank) {
    unsigned d;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(d) : "r"(smem_u32(ptr)), "r"(rank));
    return d;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Tile load into this block's shared memory whose bytes are counted by a barrier that may live in
// the other block of the pair (`bar_cluster_addr`: a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                 unsigned bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
            smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_acc, unsigned long long adesc,
                                               unsigned long long bdesc, unsigned idesc, bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_acc),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"((unsigned)accumulate)
        : "memory");
}
// Arrives, once the MMAs issued so far are done, on the barrier at this offset in both blocks.
__device__ __forceinline__ void umma_commit_pair(unsigned long long* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(
            smem_u32(bar)),
        "h"((unsigned short)3)
        : "memory");
}
template <bool F32>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TCP_THREADS)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const float* __restrict__ bias, const float* residual, void* out, int ldo, int M,
                         int N, int K, int bn, int mode, int* status) {
    const unsigned a_bytes = 256 * TC_BK * 2, w_bytes = (unsigned)(bn / 2) * TC_BK * 2;
    const unsigned stage_bytes = a_bytes + w_bytes;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ TcPairShared sh;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_block_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int k_slices = (K + TC_BK - 1) / TC_BK;
    const int tiles_m = (M + TCP_ROWS - 1) / TCP_ROWS, tiles_n = (N + bn - 1) / bn;
    const int n_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TCP_STAGES; ++s) {
            tc_mbar_init(&sh.full[s], 1);
            tc_mbar_init(&sh.empty[s], 1);
        }
        tc_mbar_init(&sh.acc_full, 1);
        tc_mbar_init(&sh.acc_empty, 2 * TCP_EPI_WARPS);  // the epilogue warps of both blocks
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == TCP_EPI_WARPS + 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         smem_u32(&sh.tmem_base)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_barrier();                                  // the peer's barriers exist from here on
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = sh.tmem_base;

    if (warp == TCP_EPI_WARPS) {
        // ---------------- producer (in both blocks)
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            for (int tile = pair; tile < n_tiles && alive; tile += n_pairs) {
                const int m0 = (tile % tiles_m) * TCP_ROWS + 128 * (int)rank;
                const int n0 = (tile / tiles_m) * bn + (bn / 2) * (int)rank;
                for (int ks = 0; ks < k_slices; ++ks, ++it) {
                    const int s = it % TCP_STAGES;
                    alive = tc_mbar_wait(&sh.empty[s], ((unsigned)(it / TCP_STAGES) & 1) ^ 1, status);
                    if (!alive) break;
                    if (rank == 0) tc_mbar_expect_tx(&sh.full[s], 2 * stage_bytes);
                    const unsigned bar = shared_of_rank(&sh.full[s], 0);
                    unsigned char* a_tile = tiles + (size_t)s * stage_bytes;
                    tma_load_2d_pair(a_tile, &map_a, ks * TC_BK, m0, bar);
                    tma_load_2d_pair(a_tile + 128 * TC_BK * 2, &map_a, ks * TC_BK, m0 + 256, bar);
                    tma_load_2d_pair(a_tile + a_bytes, &map_w, ks * TC_BK, n0, bar);
                }
            }
            if (rank == 0)                                // nothing stays in flight (the MMAs read both blocks' stages)
                for (int j = max(0, it - TCP_STAGES); j < it; ++j)
                    if (!tc_mbar_wait(&sh.full[j % TCP_STAGES], (unsigned)(j / TCP_STAGES) & 1, status)) break;
        }
    } else if (warp == TCP_EPI_WARPS + 1) {
        // ---------------- MMA issuer of the pair: rows 0-255 of the tile into columns [0, bn), rows
        // 256-511 into [256, 256 + bn) of both blocks' tensor memory
        if (lane == 0 && rank == 0) {
            const unsigned idesc = umma_idesc(256, bn);
            int it = 0, local = 0;
            bool alive = true;
            for (int tile = pair; tile < n_tiles && alive; tile += n_pairs, ++local) {
                alive = tc_mbar_wait(&sh.acc_empty, ((unsigned)local & 1) ^ 1, status);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                for (int ks = 0; ks < k_slices; ++ks, ++it) {
                    const int s = it % TCP_STAGES;
                    alive = tc_mbar_wait(&sh.full[s], (unsigned)(it / TCP_STAGES) & 1, status);
                    if (!alive) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned char* a_tile = tiles + (size_t)s * stage_bytes;
                    const unsigned long long adesc_lo = umma_desc(a_tile);
                    const unsigned long long adesc_hi = umma_desc(a_tile + 128 * TC_BK * 2);
                    const unsigned long long bdesc = umma_desc(a_tile + a_bytes);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {
                        umma_bf16_pair(tmem_base, adesc_lo + 2 * k, bdesc + 2 * k, idesc, (ks | k) != 0);
                        umma_bf16_pair(tmem_base + 256, adesc_hi + 2 * k, bdesc + 2 * k, idesc, (ks | k) != 0);
                    }
                    umma_commit_pair(&sh.empty[s]);
                }
                if (alive) umma_commit_pair(&sh.acc_full);
            }
        }
    } else {
        // ---------------- epilogue: warp w -> accumulator w / 4, lane quarter w % 4 of this block's half
        const int half = (warp >> 2) & 1, quarter = warp & 3, c_first = 32 * (warp >> 3);
        const unsigned free_bar = shared_of_rank(&sh.acc_empty, 0);
        unsigned char* stage = tiles + (size_t)TCP_STAGES * stage_bytes + (size_t)warp * 4096;
        int local = 0;
        for (int tile = pair; tile < n_tiles; tile += n_pairs, ++local) {
            const int m0 = (tile % tiles_m) * TCP_ROWS, n0 = (tile / tiles_m) * bn;
            const int row0 = m0 + 256 * half + 128 * (int)rank + 32 * quarter;
            const unsigned tbase = tmem_base + (unsigned)half * 256 + ((unsigned)(32 * quarter) << 16);
            EpilogueLane<F32> mine;
            mine.prefetch(bias, residual, out, ldo, row0, n0, c_first, bn, M, N, mode, lane);
            if (!tc_mbar_wait(&sh.acc_full, (unsigned)local & 1, status)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            mine.drain(tbase, row0, n0, c_first, bn, bias, residual, out, ldo, M, N, mode, stage, lane, free_bar);
        }
    }
    // ---------------- teardown: neither block leaves while the other may still touch its memory
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_barrier();
    if (warp == TCP_EPI_WARPS + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512)
                     : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) == cudaSuccess &&
            query == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// A [rows, K] bfloat16 matrix with `ld` elements between rows, cut into boxes of box_rows x 64.
// Encoding a map costs the host a few microseconds and a step launches some hundred products, most of
// them on the same weight matrices and the same activation buffers as the step before: maps are kept
// by what they describe (address, extents, row stride, box) and encoded once. A map holds no reference
// to the memory: a stale entry whose address now holds another tensor of the same extents describes
// that tensor just as well.
struct MapKey {
    const void* base;
    long long rows, K, ld;
    int box_rows;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows;
    }
};

struct MapSlot {
    MapKey key;
    CUtensorMap map;
    bool used;
};

constexpr int MAP_CACHE_SLOTS = 4096;           // a power of two
MapSlot g_map_cache[MAP_CACHE_SLOTS];
std::mutex g_map_cache_lock;

}  // namespace

int mx_tensor_map_2d(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
    const MapKey key = {base, rows, K, ld, box_rows};
    unsigned long long h = (unsigned long long)(size_t)base * 0x9E3779B97F4A7C15ull;
    h ^= (unsigned long long)rows * 0xC2B2AE3D27D4EB4Full + (unsigned long long)K * 0x165667B19E3779F9ull +
         (unsigned long long)ld * 0x27D4EB2F165667C5ull + (unsigned long long)box_rows;
    h ^= h >> 29;
    std::lock_guard<std::mutex> guard(g_map_cache_lock);
    MapSlot& slot = g_map_cache[h & (MAP_CACHE_SLOTS - 1)];
    if (slot.used && slot.key == key) {
        *map = slot.map;
        return MX_OK;
    }
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) MX_REFUSE("tcgen05 gemm: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) MX_REFUSE("tcgen05 gemm: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    slot.key = key;
    slot.map = *map;
    slot.used = true;
    return MX_OK;
}

namespace {

// Set by mx_gemm_tcgen05_force_tiles (0: the kernel is chosen by shape).
int g_forced_tile_rows = 0;

// The tile width that needs the fewest rounds of work per SM: the time of a product is about
// (rounds of tiles per SM) x (tile width + a fixed cost per tile).
int pick_tile_width(int M, int N, int n_sm, int tile_rows) {
    const long long tiles_m = (M + tile_rows - 1) / tile_rows;
    int best = 256;
    long long best_cost = -1;
    for (int bn = 256; bn >= 32; bn -= 16) {
        const long long tiles = tiles_m * ((N + bn - 1) / bn);
        const long long rounds = (tiles + n_sm - 1) / n_sm;
        const long long cost = rounds * (bn + (tile_rows == 128 ? 24 : 48));   // + a tile's fixed cost
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

int sm_count() {
    static int count = 0;
    if (count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
        if (count <= 0) count = 148;
    }
    return count;
}

// MATRICXON_GEMM_SPLIT_K=0 keeps every tile's K in one block (the parts of a split K meet in the output
// through additions at the memory side, whose order is not fixed: sums may differ in the last bit from
// run to run).
bool split_k_allowed() {
    static int allowed = -1;
    if (allowed < 0) {
        const char* env = getenv("MATRICXON_GEMM_SPLIT_K");
        allowed = (env != nullptr && env[0] == '0') ? 0 : 1;
    }
    return allowed == 1;
}

// Tile width and number of parts of K for the 256-row kernel when K may be split: the pair with the least
// estimated time. A block's slice of K costs the slower of its loads ((256 + bn) x 128 bytes at about 100
// bytes a nanosecond per SM) and its products; a work item ends with an epilogue; items run in rounds.
void pick_width_and_split(int M, int N, int K, int n_sm, int* best_bn, int* best_splits) {
    const long long tiles_m = (M + TCW_BM - 1) / TCW_BM;
    const int k_slices = (K + TC_BK - 1) / TC_BK;
    double best = -1.0;
    for (int bn = 256; bn >= 64; bn -= 16) {
        const long long tiles = tiles_m * ((N + bn - 1) / bn);
        for (int splits = 1; splits <= 16; ++splits) {
            const int per = (k_slices + splits - 1) / splits;
            if (per < 4 && splits > 1) break;
            if ((long long)(splits - 1) * per >= k_slices) continue;          // a part without slices
            const long long rounds = (tiles * splits + n_sm - 1) / n_sm;
            const double load_ns = (256.0 + bn) * 1.28, mma_ns = bn * 2.1;
            const double item_ns = per * (load_ns > mma_ns ? load_ns : mma_ns) + 2000.0 + bn * 25.0;
            const double cost = rounds * item_ns;
            if (best < 0 || cost < best) { best = cost; *best_bn = bn; *best_splits = splits; }
        }
    }
}

// How many pairs of SMs the pair kernel can hold at once with its largest tile (0: it cannot run).
int pair_count() {
    static int count = -1;
    if (count < 0) {
        const size_t most = (size_t)TCP_STAGES * (256 + 128) * TC_BK * 2 + TCP_STAGING + 1024;
        count = 0;
        if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)most) == cudaSuccess &&
            cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)most) == cudaSuccess) {
            cudaLaunchConfig_t config = {};
            config.gridDim = dim3(2 * sm_count());
            config.blockDim = dim3(TCP_THREADS);
            config.dynamicSmemBytes = most;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tcgen05_pair_kernel<true>, &config) == cudaSuccess)
                count = clusters;
        }
        cudaGetLastError();
    }
    return count;
}

}  // namespace

// Forces the 128-, 256- or 512-row kernel where the shape allows it (0 gives the choice back to the
// shape): tests run all three on the same product.
extern "C" int mx_gemm_tcgen05_force_tiles(int rows) {
    if (rows != 0 && rows != 128 && rows != 256 && rows != 512)
        MX_REFUSE("tcgen05 gemm: tiles of %d rows do not exist (128, 256, 512, or 0 for the shape's own)", rows);
    g_forced_tile_rows = rows;
    return MX_OK;
}

extern "C" int mx_gemm_tcgen05(const void* A, const void* W, const float* bias, const float* residual,
                               void* out, int out_dtype, int M, int N, int K, int lda, int ldw, int ldo,
                               int mode, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return MX_OK;
    if (K <= 0 || K % 8 != 0) MX_REFUSE("tcgen05 gemm: K = %d is not a positive multiple of 8", K);
    if (lda % 8 != 0 || ldw % 8 != 0)
        MX_REFUSE("tcgen05 gemm: row strides %d, %d are not multiples of 8 elements (16 bytes)", lda, ldw);
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) % 16 != 0)
        MX_REFUSE("tcgen05 gemm: operands must start on 16-byte boundaries");
    if (mode < 0 || mode > 3) MX_REFUSE("tcgen05 gemm: unknown epilogue mode %d", mode);
    if (mode == 2 && residual == nullptr) MX_REFUSE("tcgen05 gemm: residual mode without a residual");
    if ((mode >= 2) != (out_dtype == MX_DTYPE_F32))
        MX_REFUSE("tcgen05 gemm: epilogue mode %d does not write dtype %d", mode, out_dtype);
    if (status == nullptr) MX_REFUSE("tcgen05 gemm: needs a status word for its bounded waits");
    const int n_sm = sm_count();
    const int n_pairs = pair_count();
    const bool f32_out = mode >= 2;
    // the epilogue of the 256- and 512-row kernels moves 16-byte units (8 bytes of bfloat16 outputs)
    const bool vector_ok = (ldo * (f32_out ? 4 : 2)) % (f32_out ? 16 : 8) == 0 &&
                           reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                           (mode != 2 || reinterpret_cast<uintptr_t>(residual) % 16 == 0) &&
                           (bias == nullptr || reinterpret_cast<uintptr_t>(bias) % 16 == 0);
    // a residual added in place lets K be shared out between blocks (every part adds into the output)
    const bool may_split = mode == 2 && residual == out && vector_ok && split_k_allowed();
    // 512-row tiles on pairs of SMs from 2,048 rows on (below that its tiles are too few or too narrow: at
    // 1,024 rows the other two are a quarter faster); 256-row tiles (two accumulators per W
    // tile) from 257 rows on, or from 129 when K can be split, unless 128-row tiles give every SM four or
    // more: then the 128-row kernel's second accumulator buffer hides each tile's epilogue under the next
    // tile's products, which is worth more (c_fc at 2,048 rows: 132 us against 148 us)
    const long long tiles_128 = (long long)((M + 127) / 128) * ((N + 255) / 256);
    bool pair = M >= 2048 && vector_ok && n_pairs > 0;
    bool wide = false;
    if (!pair && vector_ok && M > 128) {
        if (may_split) {
            wide = true;
        } else if (M > 256 && tiles_128 < 4LL * n_sm) {
            // both kernels are bound by what a block loads per slice of K: rounds x (tile rows + tile width)
            const int bn_128 = pick_tile_width(M, N, n_sm, TC_BM), bn_256 = pick_tile_width(M, N, n_sm, TCW_BM);
            const long long t_128 = (long long)((M + 127) / 128) * ((N + bn_128 - 1) / bn_128);
            const long long t_256 = (long long)((M + 255) / 256) * ((N + bn_256 - 1) / bn_256);
            // (the 128-row kernel keeps four stages in flight and hides all epilogues but the last under the
            // next tile's products; the 256-row kernel pays for each: measured at 512-1,536 rows)
            const long long cost_128 = ((t_128 + n_sm - 1) / n_sm) * ((TC_BM + bn_128) * 9 / 10 + 32) + bn_128 / 4;
            const long long cost_256 = ((t_256 + n_sm - 1) / n_sm) * (TCW_BM + bn_256 + 32 + bn_256 / 2);
            wide = cost_256 <= cost_128;
        }
    }
    if (g_forced_tile_rows != 0) {       // mx_gemm_tcgen05_force_tiles: tests run every kernel on the same product
        const int rows = g_forced_tile_rows;
        if (rows == 128) { wide = false; pair = false; }
        if (rows == 256 && vector_ok) { wide = true; pair = false; }
        if (rows == 512 && vector_ok && n_pairs > 0) { pair = true; wide = false; }
    }
    static bool attribute_set = false;
    if (!attribute_set) {
        const size_t most = 226 * 1024;
        const size_t most_wide = (size_t)TCW_STAGES * (TCW_BM + 256) * TC_BK * 2 + TCW_STAGING + 1024;
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)most);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)most);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_tcgen05_wide_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)most_wide);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_tcgen05_wide_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)most_wide);
        if (e != cudaSuccess) MX_REFUSE("tcgen05 gemm: cannot reserve %zu bytes of shared memory", most_wide);
        attribute_set = true;
    }
    if (pair) {
        const int bn = pick_tile_width(M, N, n_pairs, TCP_ROWS);
        CUtensorMap map_a, map_w;
        int rc = mx_tensor_map_2d(&map_a, A, M, K, lda, 128);
        if (rc != MX_OK) return rc;
        rc = mx_tensor_map_2d(&map_w, W, N, K, ldw, bn / 2);
        if (rc != MX_OK) return rc;
        const size_t smem = (size_t)TCP_STAGES * (256 + bn / 2) * TC_BK * 2 + TCP_STAGING + 1024;
        const long long tiles = (long long)((M + TCP_ROWS - 1) / TCP_ROWS) * ((N + bn - 1) / bn);
        const int grid = 2 * (int)(tiles < n_pairs ? tiles : n_pairs);
        if (f32_out)
            gemm_tcgen05_pair_kernel<true><<<grid, TCP_THREADS, smem, stream>>>(map_a, map_w, bias, residual, out,
                                                                                ldo, M, N, K, bn, mode, status);
        else
            gemm_tcgen05_pair_kernel<false><<<grid, TCP_THREADS, smem, stream>>>(map_a, map_w, bias, residual, out,
                                                                                 ldo, M, N, K, bn, mode, status);
        return mx_launch_status();
    }
    if (wide) {
        int bn = pick_tile_width(M, N, n_sm, TCW_BM), k_splits = 1;
        if (may_split) pick_width_and_split(M, N, K, n_sm, &bn, &k_splits);
        CUtensorMap map_a, map_w;
        int rc = mx_tensor_map_2d(&map_a, A, M, K, lda, TCW_BM);
        if (rc != MX_OK) return rc;
        rc = mx_tensor_map_2d(&map_w, W, N, K, ldw, bn);
        if (rc != MX_OK) return rc;
        const size_t smem = (size_t)TCW_STAGES * (TCW_BM + bn) * TC_BK * 2 + TCW_STAGING + 1024;
        const long long items = (long long)((M + TCW_BM - 1) / TCW_BM) * ((N + bn - 1) / bn) * k_splits;
        const int grid = (int)(items < n_sm ? items : n_sm);
        if (f32_out)
            gemm_tcgen05_wide_kernel<true><<<grid, TCW_THREADS, smem, stream>>>(map_a, map_w, bias, residual, out,
                                                                                ldo, M, N, K, bn, mode, k_splits, status);
        else
            gemm_tcgen05_wide_kernel<false><<<grid, TCW_THREADS, smem, stream>>>(map_a, map_w, bias, residual, out,
                                                                                 ldo, M, N, K, bn, mode, k_splits, status);
        return mx_launch_status();
    }
    const int bn = pick_tile_width(M, N, n_sm, TC_BM);
    CUtensorMap map_a, map_w;
    int rc = mx_tensor_map_2d(&map_a, A, M, K, lda, TC_BM);
    if (rc != MX_OK) return rc;
    rc = mx_tensor_map_2d(&map_w, W, N, K, ldw, bn);
    if (rc != MX_OK) return rc;
    // two slices of K per stage where four such stages fit (tiles of up to 64 columns)
    int kk = 2 * TC_STAGES * (TC_BM + bn) * TC_BK * 2 + TC_STAGING + 1024 <= 226 * 1024 ? 2 : 1;
    const size_t smem = (size_t)kk * TC_STAGES * (TC_BM + bn) * TC_BK * 2 + TC_STAGING + 1024;
    const long long tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((N + bn - 1) / bn);
    const int grid = (int)(tiles < n_sm ? tiles : n_sm);
    if (f32_out)
        gemm_tcgen05_kernel<true><<<grid, TC_THREADS, smem, stream>>>(map_a, map_w, bias, residual, out, ldo, M, N, K,
                                                                      bn, mode, vector_ok ? 1 : 0, kk, status);
    else
        gemm_tcgen05_kernel<false><<<grid, TC_THREADS, smem, stream>>>(map_a, map_w, bias, residual, out, ldo, M, N, K,
                                                                       bn, mode, vector_ok ? 1 : 0, kk, status);
    return mx_launch_status();
}
