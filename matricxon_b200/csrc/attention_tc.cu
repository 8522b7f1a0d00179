// Paged attention for prompt portions on the fifth-generation tensor cores (tcgen05), bfloat16,
// head_dim 128, pages of 16 or 32 slots.
//
// Same mathematics and visibility rule as attention.cu / attention_mma.cu (query at p sees key j
// iff j <= p and (window == 0 or j > p - window); scores q.k * scale; float softmax; query head h
// reads KV head h / group), cf. app/native/src/mx_attention.c:16-68 and
// app/architectures/qwen_layers.py:12-17,94-100.
//
// A block owns, for one sequence and one KV head, T = 128 / group consecutive query tokens: the
// 128 rows of an MMA tile are the pairs (token, head in group), token-major, so all rows share
// every key. It walks the keys in chunks of 128 positions:
//   warps 8 and 10     producers: warp 8 brings the query tile once (one 4-D TMA box per half of the
//                      head dim) and per chunk the keys, warp 10 the values: TMA boxes straight out
//                      of the paged cache, one page per lane, page numbers from the block table
//                      (read once per tile into shared memory), two stages each. A key stage is
//                      free as soon as its Q K^T has run, a value stage when its P V has;
//   warp 9 (one lane)  issues S = Q K^T (tcgen05.mma, operands in swizzled shared memory,
//                      accumulator in tensor memory, three S buffers so that the scores of the
//                      next chunk exist before the softmax of this one ends) and O += P V (P read
//                      from tensor memory, V^T pages as the K-major B operand, O in tensor memory);
//   warps 0-7          softmax: two threads per row (warps w and w + 4 reach the same quarter of
//                      tensor memory), each with 64 of the chunk's 128 keys. A thread reads its
//                      scores from tensor memory (tcgen05.ld), masks the chunks that cross an edge,
//                      exchanges its maximum with its partner through shared memory, keeps a running
//                      reference maximum that only moves when the new maximum exceeds it by 2^8
//                      (then O is rescaled in tensor memory), writes P as bfloat16 over the first
//                      64 columns of the same score buffer (tcgen05.st), and at the end
//                      normalises its 64 columns of O and stores them. (One thread per row took
//                      82 us for the 2,048-token portion of the 3B sizes, two take 75: a scheduler
//                      with two softmax warps runs one's tensor-memory loads under the other's
//                      exponentials. The chunk's 16,384 exponentials alone are 1,024 cycles of the
//                      SM's special-function units, as long as its MMAs.)
// Keys beyond the newest one of the tile are not data yet: their scores are masked by selection and
// their value columns are zeroed in shared memory before the last P V (0 x NaN must not happen).
// Every mbarrier wait is bounded: a wait that runs out sets MX_STATUS_WAIT_TIMEOUT and the role
// leaves its loop, so the block always reaches the point where tensor memory is freed.
#include <cuda.h>
#include <math.h>

#include "common.cuh"

namespace {

constexpr int AT_ROWS = 128;
constexpr int AT_KEYS = 128;
constexpr int AT_HD = 128;
constexpr int AT_STAGES = 2;
constexpr int AT_SOFTMAX_WARPS = 8;                    // two per quarter of tensor memory: each takes half of a row's keys
constexpr int AT_SOFTMAX_THREADS = AT_SOFTMAX_WARPS * 32;
constexpr int AT_KEY_WARP = 8, AT_MMA_WARP = 9, AT_VALUE_WARP = 10;
constexpr int AT_THREADS = 352;                       // warps 0-7 softmax, 8 keys, 9 MMA, 10 values
constexpr unsigned AT_SPIN = 1u << 18;
constexpr int AT_TILE = AT_ROWS * 64 * 2;            // bytes of a [128][64] bfloat16 half tile
constexpr int AT_SBUF = 3;                            // score buffers in tensor memory: 3 x 128 columns, then O
constexpr int AT_TABLE = 1024;                        // block-table entries of a tile kept in shared memory
constexpr float AT_JUMP = 8.f;                        // log2 of the growth the reference maximum tolerates

struct AtShared {
    unsigned long long q_full;
    unsigned long long k_full[AT_STAGES], v_full[AT_STAGES];
    // three S buffers (P of a chunk overwrites its S): Q K^T runs two chunks ahead of P V, and a softmax
    // warp may be up to two chunks ahead of another, so every barrier of a chunk is per buffer
    unsigned long long s_full[AT_SBUF], p_full[AT_SBUF];
    // completion of the P V of even and of odd chunks: the value producer, about to refill the stage of
    // chunk j - 2, and the softmax threads wait on it; with two barriers neither can fall two phases behind
    unsigned long long pv_done[2];
    unsigned tmem_base;
    int abort;                   // a softmax thread's wait ran out: all of them leave at the next exchange
};

struct AtParams {
    const int* block_tables;     // [seqs][bt_stride]
    const int* cu_q;             // [seqs + 1]
    const int* context_lens;     // [seqs]
    const int* tiles;            // [n_tiles][2]: (sequence, first token of the tile within the sequence)
    __nv_bfloat16* out;          // [tokens][out_stride]
    float* part_o;               // n_splits > 1: [tokens][heads][splits][128] unnormalised sums
    float* part_ml;              // n_splits > 1: [tokens][heads][splits][2] (maximum in natural-log units, sum)
    int n_splits;                // blockIdx.z takes every n_splits-th share of a tile's chunks of keys
    int* status;
    long long n_pages;
    int out_stride, bt_stride, n_heads, n_kv_heads, group, tokens_per_tile, page_size, page_shift, window;
    float scale_log2;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void at_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool at_try_wait(unsigned long long* bar, unsigned parity) {
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
// false: the wait ran out (status set); the caller leaves its loop
__device__ __forceinline__ bool at_wait(unsigned long long* bar, unsigned parity, int* status) {
    for (unsigned spin = 0; spin < AT_SPIN; ++spin)
        if (at_try_wait(bar, parity)) return true;
    atomicOr(status, MX_STATUS_WAIT_TIMEOUT);
    return false;
}
__device__ __forceinline__ void tma_3d(void* dst, const CUtensorMap* map, int x, int y, int z, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_4d(void* dst, const CUtensorMap* map, int x, int y, int z, int w,
                                       unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar))
        : "memory");
}
// Shared-memory operand descriptor, K-major: rows of `swizzle bytes`, groups of 8 rows `sbo` bytes apart.
__device__ __forceinline__ unsigned long long at_desc(const void* tile, unsigned sbo, unsigned layout) {
    unsigned long long desc = 0;
    desc |= (unsigned long long)((smem_u32(tile) & 0x3FFFF) >> 4);
    desc |= (unsigned long long)1 << 16;
    desc |= (unsigned long long)(sbo >> 4) << 32;
    desc |= (unsigned long long)1 << 46;                 // descriptor version of sm_100
    desc |= (unsigned long long)layout << 61;            // 2: 128-byte swizzle, 4: 64-byte, 6: 32-byte
    return desc;
}
__device__ __forceinline__ unsigned at_idesc(int m, int n) {
    unsigned d = 0;
    d |= 1u << 4;                      // accumulator format: f32
    d |= 1u << 7;                      // A format: bf16
    d |= 1u << 10;                     // B format: bf16
    d |= (unsigned)(n >> 3) << 17;
    d |= (unsigned)(m >> 4) << 24;
    return d;
}
__device__ __forceinline__ void at_mma(unsigned tmem_acc, unsigned long long adesc, unsigned long long bdesc,
                                       unsigned idesc, bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_acc),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"((unsigned)accumulate)
        : "memory");
}
// The same with the A operand in tensor memory (16-bit elements, two per 32-bit column, row = lane).
__device__ __forceinline__ void at_mma_ts(unsigned tmem_acc, unsigned tmem_a, unsigned long long bdesc, unsigned idesc,
                                          bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_acc),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"((unsigned)accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_store32_bits(unsigned taddr, const unsigned* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
        "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
        "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void at_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_load32(unsigned taddr, float* v) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_store32(unsigned taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned at_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, const AtParams p) {
    extern __shared__ __align__(1024) unsigned char at_smem_raw[];
    __shared__ AtShared sh;
    __shared__ int table_k[AT_TABLE], table_v[AT_TABLE];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(at_smem_raw) + 1023) &
                                                           ~(uintptr_t)1023);
    unsigned char* q_tile = smem;                                   // 2 halves of [128][64]
    unsigned char* k_stage = q_tile + 2 * AT_TILE;                  // per stage: 2 halves of [128 keys][64]
    unsigned char* v_stage = k_stage + AT_STAGES * 2 * AT_TILE;     // per stage: pages of [128 dims][page_size]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = p.tiles[2 * blockIdx.x], tok0 = p.tiles[2 * blockIdx.x + 1];
    const int kh = blockIdx.y;
    const int q_start = p.cu_q[seq];
    const int q_len = p.cu_q[seq + 1] - q_start;
    const int ctx = p.context_lens[seq];
    const int n_tok = min(p.tokens_per_tile, q_len - tok0);
    if (n_tok <= 0) return;                                         // nothing was allocated yet
    const int hi_tile = ctx + tok0 + n_tok - 1;
    const int lo_tile = p.window > 0 ? max(0, ctx + tok0 - p.window + 1) : 0;
    // the tile's chunks of 128 keys, and this block's share of them when the keys are split (few tiles, a
    // long context: the shares are merged by mx_attention_merge_bf16); a share may be empty
    const int first_chunk = lo_tile / AT_KEYS;
    const int all_chunks = hi_tile / AT_KEYS + 1 - first_chunk;
    const int per_split = (all_chunks + p.n_splits - 1) / p.n_splits;
    const int c_begin = first_chunk + (int)blockIdx.z * per_split;
    const int n_chunks = max(0, min(per_split, all_chunks - (int)blockIdx.z * per_split));
    if (n_chunks == 0) {                                            // an empty share: tell the merge, touch nothing else
        const int t_in = tid / p.group, h_in = tid - t_in * p.group;
        if (tid < p.tokens_per_tile * p.group && t_in < n_tok) {
            const size_t base = ((size_t)(q_start + tok0 + t_in) * p.n_heads + (size_t)(kh * p.group + h_in)) *
                                    p.n_splits + blockIdx.z;
            p.part_ml[base * 2] = -INFINITY;
            p.part_ml[base * 2 + 1] = 0.f;
        }
        return;
    }
    const int pages_per_chunk = AT_KEYS >> p.page_shift;
    const unsigned page_bytes = (unsigned)(p.page_size * AT_HD * 2);

    if (tid == 0) {
        at_mbar_init(&sh.q_full, 1);
        for (int s = 0; s < AT_STAGES; ++s) {
            at_mbar_init(&sh.k_full[s], 1);
            at_mbar_init(&sh.v_full[s], 1);
        }
        for (int b = 0; b < AT_SBUF; ++b) {
            at_mbar_init(&sh.s_full[b], 1);
            at_mbar_init(&sh.p_full[b], AT_SOFTMAX_WARPS);
        }
        at_mbar_init(&sh.pv_done[0], 1);
        at_mbar_init(&sh.pv_done[1], 1);
        sh.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    // value stages start as zeros: a page that is never fetched must not hold NaN bit patterns
    for (int i = tid; i < AT_STAGES * 2 * AT_TILE / 16; i += AT_THREADS)
        reinterpret_cast<uint4*>(v_stage)[i] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    if (warp == AT_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh.tmem_base)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = sh.tmem_base;
    const unsigned tmem_o = tmem_base + AT_SBUF * 128;

    if (warp == AT_KEY_WARP || warp == AT_VALUE_WARP) {
        // ---------------- producers: warp 4 brings the query tile and the keys, warp 6 the values, each
        // at its own pace (a key stage is free once its Q K^T is done, a value stage once its P V is);
        // lane pg owns page pg of every chunk
        const bool keys = warp == AT_KEY_WARP;
        int* table = keys ? table_k : table_v;
        const int* bt = p.block_tables + (size_t)seq * p.bt_stride;
        if (keys && lane == 0) {
            const unsigned q_bytes = (unsigned)(2 * 64 * p.group * p.tokens_per_tile * 2);   // boxes count in full
            at_expect_tx(&sh.q_full, q_bytes);
            tma_4d(q_tile, &q_map, 0, 0, kh, q_start + tok0, &sh.q_full);
            tma_4d(q_tile + AT_TILE, &q_map, 64, 0, kh, q_start + tok0, &sh.q_full);
        }
        // this tile's part of the block table, read once (entries beyond AT_TABLE stay in global memory)
        const int first_page = (c_begin * AT_KEYS) >> p.page_shift;
        const int n_table = min(n_chunks * pages_per_chunk, AT_TABLE);
        for (int i = lane; i < n_table; i += 32) {
            const int lp = first_page + i;
            table[i] = lp < p.bt_stride ? bt[lp] : -1;
        }
        __syncwarp();
        for (int j = 0; j < n_chunks; ++j) {
            const int s = j % AT_STAGES;
            unsigned long long* full = keys ? &sh.k_full[s] : &sh.v_full[s];
            bool free_now = true;
            if (lane == 0 && j >= AT_STAGES) {
                // the stage held chunk j - 2: its keys are free once that chunk's scores exist, its values
                // once that chunk's P V has run
                const int before = j - AT_STAGES;
                free_now = keys ? at_wait(&sh.s_full[before % AT_SBUF], (unsigned)(before / AT_SBUF) & 1, p.status)
                                : at_wait(&sh.pv_done[before & 1], (unsigned)(before >> 1) & 1, p.status);
            }
            if (!__shfl_sync(0xffffffffu, free_now, 0)) break;
            const int c0 = (c_begin + j) * AT_KEYS;
            long long page = -1;
            if (lane < pages_per_chunk) {
                const int key0 = c0 + lane * p.page_size;
                if (key0 <= hi_tile && key0 + p.page_size - 1 >= lo_tile) {
                    const int i = j * pages_per_chunk + lane;
                    const int lp = first_page + i;
                    page = i < AT_TABLE ? table[i] : (lp < p.bt_stride ? bt[lp] : -1);
                    if (page < 0 || page >= p.n_pages) {
                        page = -1;
                        if (keys) atomicOr(p.status, MX_STATUS_BAD_PAGE);
                    }
                }
            }
            const unsigned n_valid = __popc(__ballot_sync(0xffffffffu, page >= 0));
            if (lane == 0) at_expect_tx(full, n_valid * page_bytes);
            __syncwarp();
            if (page >= 0) {
                const int block = (int)(page * 2 * p.n_kv_heads) + kh;
                if (keys) {
                    unsigned char* ks = k_stage + (size_t)s * 2 * AT_TILE + (size_t)lane * p.page_size * 128;
                    tma_3d(ks, &k_map, 0, 0, block, full);
                    tma_3d(ks + AT_TILE, &k_map, 64, 0, block, full);
                } else {
                    tma_3d(v_stage + (size_t)s * 2 * AT_TILE + (size_t)lane * page_bytes, &v_map, 0, 0,
                           block + p.n_kv_heads, full);
                }
            }
        }
    } else if (warp == AT_MMA_WARP) {
        // ---------------- MMA issuer. One thread; everything it can know before the loop is computed
        // there, and a chunk costs it two commits: tcgen05.mma of one thread run in issue order, so the
        // Q K^T that overwrites a score buffer needs no barrier against the P V that read P from it.
        if (lane == 0) {
            const unsigned idesc = at_idesc(AT_ROWS, AT_KEYS);
            const unsigned v_layout = p.page_size == 16 ? 6u : 4u;       // 32- or 64-byte swizzle
            const unsigned v_sbo = (unsigned)(8 * p.page_size * 2);       // eight rows of one page tile
            const int steps_per_page = p.page_size / 16;
            unsigned long long q_desc[2], k_desc[AT_STAGES][2], v_desc[AT_STAGES];
            unsigned v_step[AT_KEYS / 16];                                 // where the 16 keys of step kk start
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                q_desc[half] = at_desc(q_tile + half * AT_TILE, 1024, 2);
#pragma unroll
                for (int st = 0; st < AT_STAGES; ++st)
                    k_desc[st][half] = at_desc(k_stage + (size_t)st * 2 * AT_TILE + half * AT_TILE, 1024, 2);
            }
#pragma unroll
            for (int st = 0; st < AT_STAGES; ++st) v_desc[st] = at_desc(v_stage + (size_t)st * 2 * AT_TILE, v_sbo, v_layout);
#pragma unroll
            for (int kk = 0; kk < AT_KEYS / 16; ++kk) {
                const int pg = kk / steps_per_page, within = kk - pg * steps_per_page;
                v_step[kk] = (unsigned)((pg * page_bytes) >> 4) + 2u * within;
            }
            bool alive = at_wait(&sh.q_full, 0, p.status);
            // state of the chunk whose scores are issued next (qk_*) and of the chunk whose P V is next (pv_*)
            int qk_stage = 0, qk_buf = 0;
            unsigned qk_stage_parity = 0;
            auto issue_qk = [&]() -> bool {
                if (!at_wait(&sh.k_full[qk_stage], qk_stage_parity, p.status)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned acc = tmem_base + (unsigned)qk_buf * 128;
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        at_mma(acc, q_desc[half] + 2 * k, k_desc[qk_stage][half] + 2 * k, idesc, (half | k) != 0);
                at_commit(&sh.s_full[qk_buf]);
                if (++qk_stage == AT_STAGES) {
                    qk_stage = 0;
                    qk_stage_parity ^= 1u;
                }
                if (++qk_buf == AT_SBUF) qk_buf = 0;
                return true;
            };
            if (alive) alive = issue_qk();
            int pv_stage = 0, pv_buf = 0;
            unsigned pv_stage_parity = 0, pv_buf_parity = 0;
            for (int j = 0; j < n_chunks && alive; ++j) {
                if (j + 1 < n_chunks) {           // the scores of the next chunk, before this chunk's P V
                    alive = issue_qk();
                    if (!alive) break;
                }
                if (!at_wait(&sh.p_full[pv_buf], pv_buf_parity, p.status)) break;
                if (!at_wait(&sh.v_full[pv_stage], pv_stage_parity, p.status)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned p_addr = tmem_base + (unsigned)pv_buf * 128;
#pragma unroll
                for (int kk = 0; kk < AT_KEYS / 16; ++kk)             // 16 keys per MMA: 8 columns of P
                    at_mma_ts(tmem_o, p_addr + 8 * kk, v_desc[pv_stage] + v_step[kk], idesc, (j | kk) != 0);
                at_commit(&sh.pv_done[j & 1]);
                if (++pv_stage == AT_STAGES) {
                    pv_stage = 0;
                    pv_stage_parity ^= 1u;
                }
                if (++pv_buf == AT_SBUF) {
                    pv_buf = 0;
                    pv_buf_parity ^= 1u;
                }
            }
        }
    } else {
        // ---------------- softmax and epilogue: two threads per tile row. Warps w and w + 4 reach the same
        // quarter of tensor memory; thread `row` of half `part` owns keys 64 part .. 64 part + 63 of its row
        // in every chunk and columns 64 part .. 64 part + 63 of O. The halves exchange their maxima through
        // shared memory once a chunk (a barrier of the 256 softmax threads) and their sums once at the end.
        // With two warps per scheduler one's tensor-memory loads and exponentials run under the other's.
        __shared__ float half_max[2][2][AT_ROWS], half_sum[2][AT_ROWS];
        const int part = warp >> 2, row = tid & (AT_ROWS - 1);
        const int t_in = row / p.group, h_in = row - t_in * p.group;
        const bool valid = row < p.tokens_per_tile * p.group && t_in < n_tok;
        const int pos = valid ? ctx + tok0 + t_in : -1;                 // -1: every key is masked
        const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const unsigned lane_base = (unsigned)(32 * (warp & 3)) << 16;
        float m_ref = -INFINITY, l_run = 0.f;
        bool alive = true;
        // Phases of the "P V done" barrier are consumed strictly in order (phase j completes when the
        // P V of chunk j has run); the barrier can never be more than one phase ahead of a warp that
        // has consumed every phase below j - 1 when it starts chunk j, so a parity is never ambiguous.
        int consumed = 0;
        auto pv_consumed_through = [&](int phases) {
            while (alive && consumed < phases) {
                alive = at_wait(&sh.pv_done[consumed & 1], (unsigned)(consumed >> 1) & 1, p.status);
                ++consumed;
            }
        };
        // A thread whose wait ran out keeps walking the loop without touching anything, so that every
        // barrier below is reached by all 256 threads; they leave together after the next exchange.
        for (int j = 0; j < n_chunks; ++j) {
            const int b = j % AT_SBUF, s = j % AT_STAGES;
            if (alive) alive = at_wait(&sh.s_full[b], (unsigned)(j / AT_SBUF) & 1, p.status);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            pv_consumed_through(j - 1);               // long completed: this only keeps the count in step
            alive = __all_sync(0xffffffffu, alive);   // the tensor-memory accesses below are warp-wide
            if (!alive) *reinterpret_cast<volatile int*>(&sh.abort) = 1;
            const int c0 = (c_begin + j) * AT_KEYS, k0 = c0 + 64 * part;
            // rows that belong to no token of the tile need no mask: whatever they compute is never stored,
            // and a row's output depends on that row alone
            const bool edge = __any_sync(0xffffffffu, valid && (k0 + 63 > pos || k0 < lo));
            const unsigned s_addr = tmem_base + (unsigned)b * 128 + lane_base;
            float sc[64];
            float mx = -INFINITY;
            if (alive) {
                tmem_load32(s_addr + 64 * part, sc);
                tmem_load32(s_addr + 64 * part + 32, sc + 32);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (edge) {
#pragma unroll
                    for (int c = 0; c < 64; ++c) {
                        const int key = k0 + c;
                        sc[c] = (key <= pos && key >= lo) ? sc[c] : -INFINITY;
                    }
                }
                // four chains, so that the maximum is not one chain of 64 dependent instructions
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < 64; c += 4) {
                    m4[0] = fmaxf(m4[0], sc[c]); m4[1] = fmaxf(m4[1], sc[c + 1]);
                    m4[2] = fmaxf(m4[2], sc[c + 2]); m4[3] = fmaxf(m4[3], sc[c + 3]);
                }
                mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            }
            half_max[j & 1][part][row] = mx;
            // both halves have their scores in registers from here on: P may overwrite the other half's columns
            asm volatile("bar.sync 3, 256;\n" ::: "memory");
            if (*reinterpret_cast<volatile int*>(&sh.abort)) {
                alive = false;
                break;                                  // all 256 threads see the flag after the barrier
            }
            mx = fmaxf(mx, half_max[j & 1][part ^ 1][row]) * p.scale_log2;
            const bool jump = mx > m_ref + AT_JUMP || (m_ref == -INFINITY && mx > -INFINITY);
            const float m_new = jump ? mx : m_ref;
            // O may only be touched while no P V is running: the rare rescaling waits for the previous one
            if (j > 0 && __any_sync(0xffffffffu, jump)) {
                pv_consumed_through(j);
                alive = __all_sync(0xffffffffu, alive);
                if (alive) {
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const float alpha = jump ? at_exp2(m_ref - m_new) : 1.f;     // exp2(-inf) = 0: O was 0 anyway
                    l_run *= alpha;
#pragma unroll
                    for (int piece = 0; piece < 2; ++piece) {
                        float o[32];
                        tmem_load32(tmem_o + lane_base + 64 * part + 32 * piece, o);
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] *= alpha;
                        tmem_store32(tmem_o + lane_base + 64 * part + 32 * piece, o);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                }
            }
            if (alive) {
                m_ref = m_new;
                const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
                float sum0 = 0.f, sum1 = 0.f;
                // P as bfloat16 pairs over the first 64 columns of this chunk's S buffer: this half's 64 keys
                // are columns 32 part .. 32 part + 31
                unsigned packed[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float e0 = at_exp2(fmaf(sc[2 * c], p.scale_log2, -m_use));
                    const float e1 = at_exp2(fmaf(sc[2 * c + 1], p.scale_log2, -m_use));
                    sum0 += e0;
                    sum1 += e1;
                    packed[c] = at_pack(e0, e1);
                }
                tmem_store32_bits(s_addr + 32 * part, packed);
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                l_run += sum0 + sum1;
            }
            if (j == n_chunks - 1 && c0 + AT_KEYS - 1 > hi_tile) {
                // value slots beyond the newest key hold no data yet: zero them in the stage
                if (alive) alive = at_wait(&sh.v_full[s], (unsigned)(j / AT_STAGES) & 1, p.status);
                unsigned char* vs = v_stage + (size_t)s * 2 * AT_TILE;
                const int first_bad = hi_tile + 1 - c0;                     // first key column without data
                const int row_bytes = p.page_size * 2;
                for (int item = tid; alive && item < AT_HD * (AT_KEYS - first_bad); item += AT_SOFTMAX_THREADS) {
                    const int d = item / (AT_KEYS - first_bad), col = first_bad + item % (AT_KEYS - first_bad);
                    const int pg = col >> p.page_shift, kcol = col & (p.page_size - 1);
                    // 16-byte chunk kcol / 8 of row d, moved by the 32- or 64-byte swizzle of the tile
                    const int moved = p.page_size == 16 ? ((kcol >> 3) ^ ((d >> 2) & 1)) : ((kcol >> 3) ^ ((d >> 1) & 3));
                    *reinterpret_cast<__nv_bfloat16*>(vs + (size_t)pg * page_bytes + d * row_bytes + moved * 16 +
                                                      (kcol & 7) * 2) = __float2bfloat16_rn(0.f);
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // ordinary stores, read by the MMA
                asm volatile("bar.sync 2, 256;\n" ::: "memory");            // all eight softmax warps zeroed their part
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0 && alive) at_arrive(&sh.p_full[b]);
        }
        pv_consumed_through(n_chunks);
        // the row's sum of weights: both halves hold a part
        half_sum[part][row] = l_run;
        asm volatile("bar.sync 3, 256;\n" ::: "memory");
        l_run += half_sum[part ^ 1][row];
        alive = __all_sync(0xffffffffu, alive);
        if (alive && p.n_splits > 1) {
            // a share of the keys: the unnormalised sums, the reference maximum and the sum of weights
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const size_t base = ((size_t)(q_start + tok0 + t_in) * p.n_heads + (size_t)(kh * p.group + h_in)) *
                                    p.n_splits + blockIdx.z;
            const bool any = n_chunks > 0 && l_run > 0.f;
            if (valid && part == 0) {
                p.part_ml[base * 2] = any ? m_ref * 0.6931471805599453f : -INFINITY;
                p.part_ml[base * 2 + 1] = any ? l_run : 0.f;
            }
            if (n_chunks > 0) {                                          // warp-uniform: tensor memory holds sums
#pragma unroll
                for (int piece = 0; piece < 2; ++piece) {
                    float o[32];
                    tmem_load32(tmem_o + lane_base + 64 * part + 32 * piece, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    if (valid && any) {
                        float4* dst4 = reinterpret_cast<float4*>(p.part_o + base * AT_HD + 64 * part + 32 * piece);
#pragma unroll
                        for (int c = 0; c < 32; c += 4) dst4[c / 4] = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
                    }
                }
            }
        } else if (alive) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            __nv_bfloat16* dst = p.out + (size_t)(q_start + tok0 + t_in) * p.out_stride +
                                 (size_t)(kh * p.group + h_in) * AT_HD + 64 * part;
#pragma unroll
            for (int piece = 0; piece < 2; ++piece) {
                float o[32];
                tmem_load32(tmem_o + lane_base + 64 * part + 32 * piece, o);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (valid) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8)
                        *reinterpret_cast<uint4*>(dst + 32 * piece + c) =
                            make_uint4(at_pack(o[c] * inv, o[c + 1] * inv), at_pack(o[c + 2] * inv, o[c + 3] * inv),
                                       at_pack(o[c + 4] * inv, o[c + 5] * inv), at_pack(o[c + 6] * inv, o[c + 7] * inv));
                }
            }
        }
    }
    // ---------------- teardown: every role arrives here; then tensor memory is freed
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == AT_MMA_WARP) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
AtEncodeFn at_encode_fn() {
    static AtEncodeFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) == cudaSuccess &&
            query == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<AtEncodeFn>(ptr);
    }
    return fn;
}
int at_make_map(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
    AtEncodeFn encode = at_encode_fn();
    if (encode == nullptr) MX_REFUSE("tcgen05 attention: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims,
                               strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) MX_REFUSE("tcgen05 attention: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    return MX_OK;
}

}  // namespace


// tiles: [n_tiles][2] (sequence, first token within the sequence); a tile covers
// tokens_per_tile = 128 / group tokens of that sequence. q: [n_tokens][q_stride] with query head h
// at column h * 128. cache: [n_pages][2][kv heads][page_size * 128], keys [slot][dim], values
// [dim][slot]. Every token of every listed sequence must be covered by tiles.
extern "C" int mx_attention_merge_bf16(const float* part_o, const float* part_ml, void* out, int out_stride,
                                       int n_tokens, int n_heads, int head_dim, int n_splits, cudaStream_t stream);

// n_splits > 1: every tile's keys are shared out between n_splits blocks, whose partial results go to
// `scratch` ((tokens x heads x splits) x (128 + 2) floats) and are merged by mx_attention_merge_bf16.
extern "C" int mx_paged_attention_tc_split(const void* q, int q_stride, const void* cache, long long n_pages,
                                           int page_size, const int* block_tables, int bt_stride, const int* cu_q,
                                           const int* context_lens, const int* tiles, int n_tiles, int n_tokens,
                                           int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                                           void* out, int out_stride, int n_splits, float* scratch, int* status,
                                           cudaStream_t stream) {
    if (n_tiles <= 0 || n_tokens <= 0) return MX_OK;
    if (n_splits < 1 || n_splits > 64) MX_REFUSE("tcgen05 attention: %d key splits", n_splits);
    if (n_splits > 1 && scratch == nullptr) MX_REFUSE("tcgen05 attention: key splits without scratch memory");
    if (head_dim != AT_HD) MX_REFUSE("tcgen05 attention is built for head_dim 128, not %d", head_dim);
    if (page_size != 16 && page_size != 32) MX_REFUSE("tcgen05 attention takes pages of 16 or 32 slots, not %d", page_size);
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        MX_REFUSE("attention: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    const int group = n_heads / n_kv_heads;
    if (group > AT_ROWS) MX_REFUSE("tcgen05 attention: a query group of %d heads exceeds a tile", group);
    if (q_stride % 8 != 0 || out_stride % 8 != 0 || reinterpret_cast<uintptr_t>(q) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(out) % 16 != 0 || reinterpret_cast<uintptr_t>(cache) % 16 != 0)
        MX_REFUSE("tcgen05 attention needs 16-byte aligned rows (strides %d, %d)", q_stride, out_stride);
    if (n_kv_heads > 65535) MX_REFUSE("attention: %d kv heads exceed the grid", n_kv_heads);
    if (status == nullptr) MX_REFUSE("tcgen05 attention needs a status word for its bounded waits");
    if (n_pages * 2 * n_kv_heads > 0x7fffffffLL) MX_REFUSE("tcgen05 attention: the cache has too many pages for a TMA coordinate");
    const int tokens_per_tile = AT_ROWS / group;

    CUtensorMap q_map, k_map, v_map;
    {
        const cuuint64_t dims[4] = {(cuuint64_t)AT_HD, (cuuint64_t)group, (cuuint64_t)n_kv_heads, (cuuint64_t)n_tokens};
        const cuuint64_t strides[3] = {(cuuint64_t)AT_HD * 2, (cuuint64_t)group * AT_HD * 2, (cuuint64_t)q_stride * 2};
        const cuuint32_t box[4] = {64, (cuuint32_t)group, 1, (cuuint32_t)tokens_per_tile};
        const int rc = at_make_map(&q_map, q, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != MX_OK) return rc;
    }
    const cuuint64_t blocks = (cuuint64_t)n_pages * 2 * n_kv_heads;
    {
        const cuuint64_t dims[3] = {(cuuint64_t)AT_HD, (cuuint64_t)page_size, blocks};
        const cuuint64_t strides[2] = {(cuuint64_t)AT_HD * 2, (cuuint64_t)page_size * AT_HD * 2};
        const cuuint32_t box[3] = {64, (cuuint32_t)page_size, 1};
        const int rc = at_make_map(&k_map, cache, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != MX_OK) return rc;
    }
    {
        const cuuint64_t dims[3] = {(cuuint64_t)page_size, (cuuint64_t)AT_HD, blocks};
        const cuuint64_t strides[2] = {(cuuint64_t)page_size * 2, (cuuint64_t)page_size * AT_HD * 2};
        const cuuint32_t box[3] = {(cuuint32_t)page_size, (cuuint32_t)AT_HD, 1};
        const int rc = at_make_map(&v_map, cache, 3, dims, strides, box,
                                   page_size == 16 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc != MX_OK) return rc;
    }
    AtParams p;
    p.block_tables = block_tables; p.cu_q = cu_q; p.context_lens = context_lens; p.tiles = tiles;
    p.out = (__nv_bfloat16*)out; p.status = status; p.n_pages = n_pages; p.out_stride = out_stride;
    p.bt_stride = bt_stride; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.group = group;
    p.tokens_per_tile = tokens_per_tile; p.page_size = page_size; p.page_shift = page_size == 16 ? 4 : 5;
    p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
    p.n_splits = n_splits;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (size_t)n_tokens * n_heads * n_splits * AT_HD : nullptr;
    const size_t smem = (size_t)(2 + 2 * AT_STAGES * 2) * AT_TILE + 1024;
    static bool attribute_set = false;
    if (!attribute_set) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) MX_REFUSE("tcgen05 attention: cannot reserve %zu bytes of shared memory", smem);
        attribute_set = true;
    }
    attention_tc_kernel<<<dim3(n_tiles, n_kv_heads, n_splits), AT_THREADS, smem, stream>>>(q_map, k_map, v_map, p);
    const int rc = mx_launch_status();
    if (rc != MX_OK || n_splits == 1) return rc;
    return mx_attention_merge_bf16(p.part_o, p.part_ml, out, out_stride, n_tokens, n_heads, AT_HD, n_splits, stream);
}

extern "C" int mx_paged_attention_tc(const void* q, int q_stride, const void* cache, long long n_pages,
                                     int page_size, const int* block_tables, int bt_stride, const int* cu_q,
                                     const int* context_lens, const int* tiles, int n_tiles, int n_tokens,
                                     int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                                     void* out, int out_stride, int* status, cudaStream_t stream) {
    return mx_paged_attention_tc_split(q, q_stride, cache, n_pages, page_size, block_tables, bt_stride, cu_q,
                                       context_lens, tiles, n_tiles, n_tokens, n_heads, n_kv_heads, head_dim, window,
                                       scale, out, out_stride, 1, nullptr, status, stream);
}
