// Device-side pieces that every tcgen05 / TMA kernel of this library uses: mbarriers with bounded
// waits, tiled TMA loads, shared-memory and instruction descriptors of kind::f16 products, the
// commit and the tensor-memory loads. Included by the kernel files; everything is file-local.
#pragma once

#include <cuda.h>

#include "common.cuh"

// A [rows, K] bfloat16 matrix with `ld` elements between rows, cut into boxes of box_rows x 64
// (128-byte swizzle). Encoded once per distinct operand and kept (gemm_tcgen05.cu).
int mx_tensor_map_2d(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows);

namespace {

constexpr int TC_BK = 64;              // 64 bf16 = 128 bytes = one swizzle row
constexpr int TC_SPIN_LIMIT = 1 << 22;

__device__ __forceinline__ unsigned smem_u32(const void* ptr) {
    return (unsigned)__cvta_generic_to_shared(ptr);
}
__device__ __forceinline__ void tc_mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool tc_mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Returns false when the wait ran out (the status word is set; the caller carries on).
__device__ __forceinline__ bool tc_mbar_wait(unsigned long long* bar, unsigned parity, int* status) {
    for (int spin = 0; spin < TC_SPIN_LIMIT; ++spin)
        if (tc_mbar_try_wait(bar, parity)) return true;
    atomicOr(status, MX_STATUS_WAIT_TIMEOUT);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y,
                                            unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
            smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, groups of
// eight rows 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc(const void* smem_tile) {
    unsigned long long desc = 0;
    desc |= (unsigned long long)((smem_u32(smem_tile) & 0x3FFFF) >> 4);        // start address
    desc |= (unsigned long long)1 << 16;                                       // leading offset (unused here)
    desc |= (unsigned long long)(1024 >> 4) << 32;                             // stride between 8-row groups
    desc |= (unsigned long long)1 << 46;                                       // descriptor version of sm_100
    desc |= (unsigned long long)2 << 61;                                       // SWIZZLE_128B
    return desc;
}

// Instruction descriptor of kind::f16: bf16 x bf16 -> f32, both operands K-major, M x N tile.
__device__ __forceinline__ unsigned umma_idesc(int m, int n) {
    unsigned d = 0;
    d |= 1u << 4;                      // accumulator format: f32
    d |= 1u << 7;                      // A format: bf16
    d |= 1u << 10;                     // B format: bf16
    d |= (unsigned)(n >> 3) << 17;
    d |= (unsigned)(m >> 4) << 24;
    return d;
}

__device__ __forceinline__ void umma_bf16(unsigned tmem_acc, unsigned long long adesc,
                                          unsigned long long bdesc, unsigned idesc, bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_acc),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"((unsigned)accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tc_mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_load16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}


// ---- issue by one lane of a warp that runs its loop as a whole -------------------------------------
// tcgen05.mma, tcgen05.commit and the TMA loads take their descriptors and addresses from uniform
// registers. A role written as `if (lane == 0) { loop }` runs in divergent code, where the compiler
// has no uniform registers: every operand of every instruction is moved over one by one, and a
// tcgen05.mma then costs its issuing thread about 90 cycles whatever its shape (measured on B200: 89
// cycles for M = 128 and N = 16 .. 128). When the WHOLE warp runs the loop (warp index made uniform
// by a shuffle, all lanes wait on the barriers) and only the instruction itself is predicated on
// elect.sync, the same product costs 39 cycles at N = 16 and 64 at N = 128, i.e. what the tensor
// pipe takes. The helpers below are that form; all 32 lanes must call them together.
__device__ __forceinline__ int uniform_warp_index() { return __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0); }

__device__ __forceinline__ void umma_bf16_elect(unsigned tmem_acc, unsigned long long adesc,
                                                unsigned long long bdesc, unsigned idesc, bool accumulate) {
    asm volatile(
        "{\n.reg .pred p, q;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_acc),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"((unsigned)accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit_elect(unsigned long long* bar) {
    asm volatile(
        "{\n.reg .pred q;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n" ::"r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tc_mbar_expect_tx_elect(unsigned long long* bar, unsigned bytes) {
    asm volatile(
        "{\n.reg .pred q;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n}\n" ::"r"(smem_u32(bar)), "r"(bytes)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d_elect(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                  unsigned long long* bar) {
    asm volatile(
        "{\n.reg .pred q;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "@q cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n}\n" ::"r"(
            smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// A bounded wait by a whole warp: every lane polls; the status word is set by one of them.
__device__ __forceinline__ bool tc_mbar_wait_warp(unsigned long long* bar, unsigned parity, int* status) {
    for (int spin = 0; spin < TC_SPIN_LIMIT; ++spin)
        if (tc_mbar_try_wait(bar, parity)) return true;
    if ((threadIdx.x & 31) == 0) atomicOr(status, MX_STATUS_WAIT_TIMEOUT);
    return false;
}

}  // namespace
