// A whole decode step (one new token per sequence, at most 16 sequences) as ONE persistent
// kernel: embedding, every layer (LayerNorm, QKV product with rotation and cache write, paged
// attention, output product, LayerNorm, up product with GELU, down product), the final norm and
// the head.
//
// Why. A decode step reads every weight once and little else; run as separate kernels, each
// product pays a launch gap and a first-load latency during which HBM is idle (about 3 us of
// the 6-15 us a product takes at these sizes). Here one block per SM stays resident and the
// step is a stream:
//   * warp 8 of every block is a producer. It walks the block's share of the step in order
//     (16 weight rows x 512 columns per chunk, or one 32-key chunk of cached keys and values)
//     and brings each chunk into a ring of shared-memory slots with bulk asynchronous copies
//     (cp.async.bulk, completion counted on an mbarrier). It only waits for a free slot, so it
//     runs ahead of the arithmetic, across phase boundaries and layers: HBM stays busy while
//     the other warps wait at a grid barrier. The one thing it waits for is the barrier that
//     publishes this step's own keys and values before it copies the page that holds them.
//   * warps 0-7 are consumers. Per phase they stage the (normalised) activations of all rows
//     in shared memory, multiply chunk after chunk with mma.sync.m16n8k16 (weights on the M
//     side, rows on the N side, as in gemm_skinny.cu and with the same order of additions),
//     reduce across the warps in a fixed order, apply the epilogue and write the result.
//   * phases are separated by a grid barrier (one atomic counter; the kernel is launched
//     cooperatively so all blocks are resident). Everything that crosses blocks goes through
//     L2 (ld.global.cg) after the barrier.
// LayerNorm statistics: the block that writes a slice of the residual stream also writes
// (count, mean, M2) of that slice per row; the readers combine the slices' statistics in a fixed
// order (Chan's parallel formula), so the statistics are float and need no second pass.
// Attention: a block takes a (row, KV head, split of the keys); each consumer warp takes every
// eighth chunk with the arithmetic of attention_mma.cu (narrow tiles), the warps' partial
// results are combined in shared memory and written as unnormalised partials; a short phase
// merges the splits.
// Every wait (mbarrier, grid barrier) is bounded; when one runs out the block sets
// MX_STATUS_WAIT_TIMEOUT, all later waits of the grid return at once and the kernel ends with
// void results. The block's own copies in flight are waited for before it exits.
//
// Mathematics as in the separate kernels: app/architectures/starcoder2_layers.py:19-23,45-68
// (block), app/architectures/qwen_layers.py:50-102 (attention), app/architectures/rope.py:152-169.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <cuda.h>

#include "common.cuh"
#include "decode_fused.h"

namespace {

constexpr int DF_WARPS = 8;
constexpr int DF_CONSUMERS = DF_WARPS * 32;
constexpr int DF_PRODUCERS = 1;                       // producer warps: chunk number q is issued by warp q % 4
constexpr int DF_THREADS = DF_CONSUMERS + 32 * DF_PRODUCERS;
constexpr int DF_KC = 512;                           // columns of a weight chunk
constexpr int DF_BOX_COLS = 256;                     // a chunk arrives as two TMA boxes of 256 columns
constexpr int DF_BOX_BYTES = 16 * DF_BOX_COLS * 2;   // 8192: 16 rows of one box
constexpr int DF_SLOT_BYTES = 17408;                 // two boxes, or 32 keys + 32 values of 128 dims, or
                                                     // 4096 floats of LayerNorm scale, with room to spare
constexpr int DF_UMAX = 2;                           // units accumulated side by side when K is staged in slices
constexpr int DF_STAT_COLS = 64;                     // residual features one block may write per phase
constexpr int DF_CHUNK = 32;                         // keys per attention chunk
constexpr unsigned DF_SPIN_LIMIT = 1u << 22;         // polls of an mbarrier
constexpr unsigned DF_GRID_SPIN_LIMIT = 1u << 21;    // polls of the grid counter (an L2 round trip each)

enum { MODE_QKV = 0, MODE_RESIDUAL = 1, MODE_GELU = 2, MODE_LOGITS = 3 };

// Cycle counters per block for tuning (compile with -DDF_PROFILE): where warp 0 and the producer
// spend their time. Read with mx_decode_fused_profile.
enum { PF_COMBINE = 0, PF_CHUNKS, PF_GRID, PF_STAGE, PF_FINISH, PF_ATTENTION, PF_MERGE, PF_WAIT_EMPTY,
       PF_WAIT_CHUNK, PF_TOTAL, PF_PRODUCER_TOTAL, PF_WAIT_KV, PF_COUNT = 16 };
#ifdef DF_PROFILE
__device__ unsigned long long g_profile[256][PF_COUNT];
__device__ __forceinline__ long long cycles_now() {
    long long t;
    asm volatile("mov.u64 %0, %%clock64;\n" : "=l"(t));
    return t;
}
struct Timer {
    int which; bool on; long long t0;
    __device__ Timer(int w, bool enabled) : which(w), on(enabled) { t0 = cycles_now(); }
    __device__ ~Timer() { if (on) g_profile[blockIdx.x][which] += (unsigned long long)(cycles_now() - t0); }
};
#define DF_TIME(which, enabled) Timer df_timer_##which(which, enabled)
#else
#define DF_TIME(which, enabled)
#endif

// ------------------------------------------------------------------ small device helpers
__device__ __forceinline__ unsigned smem_addr(const void* ptr) { return (unsigned)__cvta_generic_to_shared(ptr); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_copy(void* smem_dst, const void* gmem_src, unsigned bytes,
                                          unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
            smem_addr(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}
// One box of a tensor map (in device memory) to shared memory: columns from x, rows from y.
__device__ __forceinline__ void tma_box(void* smem_dst, const void* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
            smem_addr(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
        : "memory");
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async;\n" ::: "memory"); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(DF_CONSUMERS) : "memory"); }

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Loads of what other blocks wrote earlier in this launch: from L2, never from this SM's L1.
__device__ __forceinline__ float ld_cg(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];\n" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float4 ld_cg4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float2 ld_cg2(const float* p) {
    float2 v;
    asm volatile("ld.global.cg.v2.f32 {%0,%1}, [%2];\n" : "=f"(v.x), "=f"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// ------------------------------------------------------------------ the block's state
struct Cx {
    unsigned char* ring;
    __nv_bfloat16* xs;               // activation stage [8 MB rows][x_pitch]
    float* red;                      // [warp][16][8 MB]
    float* stat_vals;                // [8 MB rows][DF_STAT_COLS]
    float* row_stats;                // [16][2] mean, 1/std
    unsigned long long* full;
    unsigned long long* empty;
    unsigned long long* xs_bar;      // completion of the bulk copies into the stage
    unsigned xs_phase;
    volatile int* abort_flag;
    int* status;
    int slots, x_pitch, x_cols;
    int slot;                        // ring position of the next chunk
    unsigned round;                  // how many times the ring wrapped
    unsigned epoch;                  // grid barriers passed
    int tid, warp, lane, g, t;
    int pid;                         // producer warps: which of them
    unsigned seq;                    // producer warps: chunks passed so far
#ifdef DF_PROFILE
    long long t_wait_full, t_wait_empty;   // cycles, kept in registers and written once at the end
#endif
};

// Every producer warp walks the whole sequence of chunks; each chunk is issued by one of them.
__device__ __forceinline__ bool my_chunk(Cx& cx) { return (cx.seq++ & (DF_PRODUCERS - 1)) == (unsigned)cx.pid; }

__device__ __forceinline__ void ring_advance(Cx& cx) {
    if (++cx.slot == cx.slots) {
        cx.slot = 0;
        ++cx.round;
    }
}
__device__ __forceinline__ void give_up(Cx& cx) {
    *cx.abort_flag = 1;
    atomicOr(cx.status, MX_STATUS_WAIT_TIMEOUT);
}
// consumer: the chunk at the ring position has landed
// a long wait looks at the step's status word now and then: if any block of the grid gave up,
// nobody waits any more
__device__ __forceinline__ bool others_gave_up(Cx& cx, unsigned spin) {
    if ((spin & 4095u) != 4095u) return false;
    if (!(*(volatile int*)cx.status & MX_STATUS_WAIT_TIMEOUT)) return false;
    *cx.abort_flag = 1;
    return true;
}
// One lane of the warp polls; the warp's other lanes meet it at __syncwarp, which also orders
// their later reads of the slot after the lane's acquire.
__device__ __forceinline__ void poll(Cx& cx, unsigned long long* bar, unsigned parity) {
    if (cx.lane == 0 && !*cx.abort_flag) {
        bool done = false;
        for (unsigned spin = 0; spin < DF_SPIN_LIMIT && !done; ++spin) {
            done = mbar_try_wait(bar, parity);
            if (!done && others_gave_up(cx, spin)) break;
        }
        if (!done && !*cx.abort_flag) give_up(cx);
    }
    __syncwarp();
}
__device__ __forceinline__ void wait_full(Cx& cx) {
#ifdef DF_PROFILE
    const long long t0 = cycles_now();
#endif
    poll(cx, &cx.full[cx.slot], cx.round & 1u);
#ifdef DF_PROFILE
    cx.t_wait_full += cycles_now() - t0;
#endif
}
// consumer warp: done with the chunk at the ring position
__device__ __forceinline__ void release_slot(Cx& cx) {
    __syncwarp();
    if (cx.lane == 0) mbar_arrive(&cx.empty[cx.slot]);
}
// producer: the slot at the ring position may be overwritten
__device__ __forceinline__ void wait_empty(Cx& cx) {
    if (cx.round == 0) return;
#ifdef DF_PROFILE
    const long long t0 = cycles_now();
#endif
    poll(cx, &cx.empty[cx.slot], (cx.round - 1u) & 1u);
#ifdef DF_PROFILE
    cx.t_wait_empty += cycles_now() - t0;
#endif
}

// All consumer threads of all blocks meet; what they wrote before is visible to all after.
__device__ __forceinline__ void grid_barrier(const MxDfParams& p, Cx& cx) {
    DF_TIME(PF_GRID, cx.tid == 0);
    ++cx.epoch;
    consumer_sync();
    if (cx.tid == 0) {
        __threadfence();
        atomicAdd(p.barrier, 1u);
        const unsigned target = cx.epoch * (unsigned)p.grid;
        if (!*cx.abort_flag) {
            unsigned spin = 0;
            while (ld_acquire_u32(p.barrier) < target) {
                if (++spin > DF_GRID_SPIN_LIMIT) {
                    give_up(cx);
                    break;
                }
                if ((spin & 255u) == 0 && (*(volatile int*)p.status & MX_STATUS_WAIT_TIMEOUT)) {
                    *cx.abort_flag = 1;      // another block gave up: nobody waits any more
                    break;
                }
            }
        }
        __threadfence();
    }
    consumer_sync();
}
// producer: barrier number `index` (1-based) has been passed by every block
__device__ __forceinline__ void producer_wait_grid(const MxDfParams& p, Cx& cx, unsigned index) {
    DF_TIME(PF_WAIT_KV, cx.lane == 0);
    if (*cx.abort_flag) return;
    const unsigned target = index * (unsigned)p.grid;
    unsigned spin = 0;
    while (ld_acquire_u32(p.barrier) < target) {
        if (++spin > DF_GRID_SPIN_LIMIT) {
            give_up(cx);
            return;
        }
        if ((spin & 255u) == 0 && (*(volatile int*)p.status & MX_STATUS_WAIT_TIMEOUT)) {
            *cx.abort_flag = 1;
            return;
        }
    }
    fence_async_proxy();     // the copies that follow read what generic stores of other blocks wrote
}

// ------------------------------------------------------------------ the share of a block
__device__ __forceinline__ int unit_begin(int block, int n_units, int grid) {
    return (int)(((long long)block * n_units) / grid);
}
// Feature (weight row) of row r of unit u. In the QKV product a unit of a rotated head holds
// dims 8j..8j+7 and their partners at + head_dim / 2, so the rotation needs no other unit.
__device__ __forceinline__ int unit_feature(int u, int r, bool rope_map, int head_dim, int rotated_heads) {
    if (!rope_map) return 16 * u + r;
    const int per_head = head_dim >> 4;
    const int head = u / per_head, j = u - head * per_head;
    if (head < rotated_heads) return head * head_dim + 8 * j + (r < 8 ? r : (head_dim >> 1) + r - 8);
    return head * head_dim + 16 * j + r;
}

struct Gemm {
    const void* map;                 // tensor map over W
    const __nv_bfloat16* W;
    const float* bias;
    int N, K, mode;
    // activations: LayerNorm of the residual stream (ln_w != null) or a bfloat16 matrix
    const float* ln_w;
    const float* ln_b;
    float ln_eps;
    const __nv_bfloat16* src;
    int src_ld;
    const MxDfLayer* layer;          // MODE_QKV
};

// ------------------------------------------------------------------ producer
__device__ __forceinline__ void produce_gemm(const MxDfParams& p, Cx& cx, const Gemm& d) {
    const bool rope_map = d.mode == MODE_QKV;
    const int n_units = (d.N + 15) >> 4;
    const int u0 = unit_begin(blockIdx.x, n_units, p.grid), u1 = unit_begin(blockIdx.x + 1, n_units, p.grid);
    const int n_slices = (d.K + cx.x_cols - 1) / cx.x_cols;
    const int group_size = n_slices == 1 ? 1 : DF_UMAX;
    int staged = -1;
    for (int ug = u0; ug < u1; ug += group_size) {
        const int gn = min(group_size, u1 - ug);
        for (int s = 0; s < n_slices; ++s) {
            const int k_begin = s * cx.x_cols, k_end = min(d.K, k_begin + cx.x_cols);
            if (staged != s) {
                staged = s;
                // the consumers stage this slice now: LayerNorm scale and shift travel like weights
                for (int which = 0; which < 2; ++which) {
                    const float* vec = which == 0 ? d.ln_w : d.ln_b;
                    if (vec == nullptr) continue;
                    const bool mine = my_chunk(cx);
                    if (mine) wait_empty(cx);
                    if (mine && !*cx.abort_flag && cx.lane == 0) {
                        const unsigned bytes = (unsigned)((k_end - k_begin) * 4);
                        mbar_expect_tx(&cx.full[cx.slot], bytes);
                        bulk_copy(cx.ring + (size_t)cx.slot * DF_SLOT_BYTES, vec + k_begin, bytes, &cx.full[cx.slot]);
                    }
                    __syncwarp();
                    ring_advance(cx);
                }
            }
            for (int ul = 0; ul < gn; ++ul) {
                const int u = ug + ul;
                // rows of the unit: one box of 16, or (QKV) two boxes of 8 that may lie apart
                const int y0 = unit_feature(u, 0, rope_map, p.head_dim, p.n_heads + p.n_kv_heads);
                const int y1 = unit_feature(u, 8, rope_map, p.head_dim, p.n_heads + p.n_kv_heads);
                for (int k0 = k_begin; k0 < k_end; k0 += DF_KC) {
                    const bool mine = my_chunk(cx);
                    if (mine) wait_empty(cx);
                    if (mine && !*cx.abort_flag && cx.lane == 0) {
                        unsigned long long* bar = &cx.full[cx.slot];
                        unsigned char* dst = cx.ring + (size_t)cx.slot * DF_SLOT_BYTES;
                        const int halves = k0 + DF_BOX_COLS < k_end ? 2 : 1;
                        mbar_expect_tx(bar, (unsigned)(halves * DF_BOX_BYTES));      // a box counts in full
                        for (int h = 0; h < halves; ++h) {
                            if (rope_map) {
                                tma_box(dst + h * DF_BOX_BYTES, d.map, k0 + h * DF_BOX_COLS, y0, bar);
                                tma_box(dst + h * DF_BOX_BYTES + DF_BOX_BYTES / 2, d.map, k0 + h * DF_BOX_COLS, y1, bar);
                            } else {
                                tma_box(dst + h * DF_BOX_BYTES, d.map, k0 + h * DF_BOX_COLS, y0, bar);
                            }
                        }
                    }
                    __syncwarp();
                    ring_advance(cx);
                }
            }
        }
    }
}

struct AttnItem {
    int row, kh, split, seq, ctx, lo, c_begin, c_end;
};
__device__ __forceinline__ AttnItem attn_item(const MxDfParams& p, const MxDfLayer& L, int item) {
    AttnItem a;
    a.split = item % p.n_splits;
    const int rest = item / p.n_splits;
    a.kh = rest % p.n_kv_heads;
    a.row = rest / p.n_kv_heads;
    a.seq = p.tok_seq[a.row];
    a.ctx = p.context_lens[a.row];
    a.lo = L.window > 0 ? max(0, a.ctx - L.window + 1) : 0;
    if (a.seq < 0) {                   // a padding row: no keys
        a.c_begin = a.c_end = 0;
        return a;
    }
    const int first = a.lo / DF_CHUNK, last = a.ctx / DF_CHUNK;
    const int per_split = (last - first + p.n_splits) / p.n_splits;
    a.c_begin = first + a.split * per_split;
    a.c_end = min(last + 1, a.c_begin + per_split);
    if (a.c_end < a.c_begin) a.c_end = a.c_begin;
    return a;
}

template <int HD>
__device__ __forceinline__ void produce_attention(const MxDfParams& p, Cx& cx, const MxDfLayer& L, unsigned kv_barrier) {
    const int shift = p.page_size == 8 ? 3 : (p.page_size == 16 ? 4 : 5);
    const int pages = DF_CHUNK >> shift;
    const unsigned tile_bytes = (unsigned)(p.page_size * HD * 2);
    const size_t head_stride = (size_t)p.page_size * HD;
    const size_t page_stride = 2 * (size_t)p.n_kv_heads * head_stride;
    const int n_items = p.rows * p.n_kv_heads * p.n_splits;
    bool waited = false;
    for (int item = blockIdx.x; item < n_items; item += p.grid) {
        const AttnItem a = attn_item(p, L, item);
        const int* bt = p.block_tables[L.group] + (size_t)a.row * p.bt_stride[L.group];
        const __nv_bfloat16* kbase = L.cache + (size_t)a.kh * head_stride;
        const __nv_bfloat16* vbase = L.cache + (size_t)(p.n_kv_heads + a.kh) * head_stride;
        for (int ci = a.c_begin; ci < a.c_end; ++ci) {
            const int c0 = ci * DF_CHUNK;
            const bool mine = my_chunk(cx);
            if (mine) wait_empty(cx);
            // the chunk with this step's own key and value exists only after the QKV phase
            if (mine && !waited && c0 + DF_CHUNK > a.ctx) {
                producer_wait_grid(p, cx, kv_barrier);
                waited = true;
            }
            if (mine && !*cx.abort_flag) {
                unsigned char* dst = cx.ring + (size_t)cx.slot * DF_SLOT_BYTES;
                __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(dst);
                __nv_bfloat16* vs = ks + DF_CHUNK * HD;
                long long page = -1;
                if (cx.lane < pages) {
                    const int key0 = c0 + cx.lane * p.page_size;
                    if (key0 <= a.ctx && key0 + p.page_size - 1 >= a.lo) {
                        const int lp = key0 >> shift;
                        page = lp < p.bt_stride[L.group] ? bt[lp] : -1;
                        if (page < 0 || page >= L.n_pages) {
                            page = -1;
                            atomicOr(cx.status, MX_STATUS_BAD_PAGE);
                        }
                    }
                }
                const unsigned have = __ballot_sync(0xffffffffu, page >= 0);
                for (int pg = 0; pg < pages; ++pg)
                    if (!((have >> pg) & 1u)) {      // a page outside the visible range: zeros, not stale bits
                        uint4* kz = reinterpret_cast<uint4*>(ks + (size_t)pg * p.page_size * HD);
                        uint4* vz = reinterpret_cast<uint4*>(vs + (size_t)pg * p.page_size * HD);
                        for (int i = cx.lane; i < (int)(tile_bytes / 16); i += 32) {
                            kz[i] = make_uint4(0, 0, 0, 0);
                            vz[i] = make_uint4(0, 0, 0, 0);
                        }
                    }
                __syncwarp();
                unsigned long long* bar = &cx.full[cx.slot];
                if (cx.lane == 0) mbar_expect_tx(bar, __popc(have) * 2u * tile_bytes);
                __syncwarp();
                if (page >= 0) {
                    bulk_copy(ks + (size_t)cx.lane * p.page_size * HD, kbase + (size_t)page * page_stride, tile_bytes, bar);
                    bulk_copy(vs + (size_t)cx.lane * p.page_size * HD, vbase + (size_t)page * page_stride, tile_bytes, bar);
                }
            }
            ring_advance(cx);
        }
    }
}

// ------------------------------------------------------------------ consumers: statistics
// (count, mean, M2) of `count` values per row, held in stat_vals, to this block's place in the
// table [row][block].
__device__ __forceinline__ int stats_pitch(const MxDfParams& p) { return (p.grid + 31) & ~31; }
__device__ __forceinline__ void write_partial_stats(const MxDfParams& p, Cx& cx, int count) {
    consumer_sync();
    if (cx.tid < p.rows) {
        const float* v = cx.stat_vals + cx.tid * DF_STAT_COLS;
        float mean = 0.f, m2 = 0.f;
        if (count > 0) {
            for (int i = 0; i < count; ++i) mean += v[i];
            mean /= (float)count;
            for (int i = 0; i < count; ++i) m2 += (v[i] - mean) * (v[i] - mean);
        }
        *reinterpret_cast<float4*>(p.stats + ((size_t)cx.tid * stats_pitch(p) + blockIdx.x) * 4) =
            make_float4((float)count, mean, m2, 0.f);
    }
}
__device__ __forceinline__ float warp_total(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
// Mean and 1/std of every row from all blocks' partial statistics, in a fixed order: the mean is
// the weighted mean of the slices' means, the sum of squares is the slices' own plus each slice's
// count times the square of its mean's distance from the whole mean (the pairwise formula of Chan
// et al. applied to all slices at once). One warp per row, a slice per lane and round.
__device__ __forceinline__ void combine_stats(const MxDfParams& p, Cx& cx, float eps) {
    const int pitch = stats_pitch(p);
    for (int m = cx.warp; m < p.rows; m += DF_WARPS) {
        const float* row = p.stats + (size_t)m * pitch * 4;
        float4 s[8];
        float count = 0.f, weighted = 0.f;
        for (int c0 = 0; c0 < p.grid; c0 += 256) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = c0 + 32 * j + cx.lane;
                s[j] = c < p.grid ? ld_cg4(row + (size_t)c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                count += s[j].x;
                weighted += s[j].x * s[j].y;
            }
        }
        count = warp_total(count);
        const float mean = warp_total(weighted) / fmaxf(count, 1.f);
        float squares = 0.f;
        for (int c0 = 0; c0 < p.grid; c0 += 256) {
            if (p.grid > 256) {                  // more slices than one round holds: read them again
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int c = c0 + 32 * j + cx.lane;
                    s[j] = c < p.grid ? ld_cg4(row + (size_t)c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) squares += s[j].z + s[j].x * (s[j].y - mean) * (s[j].y - mean);
        }
        squares = warp_total(squares);
        if (cx.lane == 0) {
            cx.row_stats[2 * m] = mean;
            cx.row_stats[2 * m + 1] = rsqrtf(squares / fmaxf(count, 1.f) + eps);
        }
    }
    consumer_sync();
}

// ------------------------------------------------------------------ consumers: products
// Activations of one slice of K into the stage, as bfloat16 [8 MB rows][x_pitch]: thread 0 issues
// one bulk copy per row (of the attention output, of the feed-forward middle, or of the bfloat16
// copy of the residual stream) and everyone waits on the stage's own mbarrier. For a LayerNorm
// the rows are then normalised in place, in float, with the scale and shift that the producer
// sent through the ring like weights, and rounded once more.
template <int MB>
__device__ __forceinline__ void stage_activations(const MxDfParams& p, Cx& cx, const Gemm& d, int k_begin, int k_end) {
    const int cols = k_end - k_begin;
    constexpr int ROWS = 8 * MB;
    const bool norm = d.ln_w != nullptr;
    const __nv_bfloat16* src = norm ? p.xb : d.src;
    const int src_ld = norm ? p.hidden : d.src_ld;
    consumer_sync();                         // every warp is done reading what the stage held
    if (cx.tid == 0 && !*cx.abort_flag) {
        fence_async_proxy();                 // the stage was read and written by ordinary accesses so far
        mbar_expect_tx(cx.xs_bar, (unsigned)(p.rows * cols * 2));
        for (int m = 0; m < p.rows; ++m)
            bulk_copy(cx.xs + (size_t)m * cx.x_pitch, src + (size_t)m * src_ld + k_begin, (unsigned)(cols * 2),
                      cx.xs_bar);
    }
    const int c8n = cols >> 3;
    for (int idx = cx.tid; idx < (ROWS - p.rows) * c8n; idx += DF_CONSUMERS) {
        const int m = p.rows + idx / c8n, c8 = idx % c8n;
        *reinterpret_cast<uint4*>(cx.xs + (size_t)m * cx.x_pitch + 8 * c8) = make_uint4(0u, 0u, 0u, 0u);
    }
    const float* gamma = nullptr;
    const float* beta = nullptr;
    int slot_gamma = -1, slot_beta = -1;
    if (norm) {                              // scale (and shift) of this slice: the next chunks of the ring
        wait_full(cx);
        gamma = reinterpret_cast<const float*>(cx.ring + (size_t)cx.slot * DF_SLOT_BYTES);
        slot_gamma = cx.slot;
        ring_advance(cx);
        if (d.ln_b != nullptr) {
            wait_full(cx);
            beta = reinterpret_cast<const float*>(cx.ring + (size_t)cx.slot * DF_SLOT_BYTES);
            slot_beta = cx.slot;
            ring_advance(cx);
        }
    }
    poll(cx, cx.xs_bar, cx.xs_phase & 1u);
    ++cx.xs_phase;
    if (norm) {
        for (int idx = cx.tid; idx < p.rows * c8n; idx += DF_CONSUMERS) {
            const int m = idx / c8n, c8 = idx - m * c8n;
            uint4* place = reinterpret_cast<uint4*>(cx.xs + (size_t)m * cx.x_pitch + 8 * c8);
            const uint4 raw = *place;
            const float mean = cx.row_stats[2 * m], rstd = cx.row_stats[2 * m + 1];
            const unsigned words[4] = {raw.x, raw.y, raw.z, raw.w};
            unsigned out[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 pair = *reinterpret_cast<const __nv_bfloat162*>(&words[e]);
                const int k = 8 * c8 + 2 * e;
                float lo = (__low2float(pair) - mean) * rstd * gamma[k];
                float hi = (__high2float(pair) - mean) * rstd * gamma[k + 1];
                if (beta != nullptr) {
                    lo += beta[k];
                    hi += beta[k + 1];
                }
                out[e] = pack_bf16(lo, hi);
            }
            *place = make_uint4(out[0], out[1], out[2], out[3]);
        }
        __syncwarp();
        if (cx.lane == 0) {
            mbar_arrive(&cx.empty[slot_gamma]);
            if (slot_beta >= 0) mbar_arrive(&cx.empty[slot_beta]);
        }
    }
    consumer_sync();
}

template <int MB>
__device__ __forceinline__ void multiply_chunk(const Cx& cx, int col0, int k_blocks, float (&acc)[MB][4]) {
    const unsigned char* slot = cx.ring + (size_t)cx.slot * DF_SLOT_BYTES;
    for (int kb = cx.warp; kb < k_blocks; kb += DF_WARPS) {
        // box kb / 8 holds columns 256 (kb / 8) ...: rows of 512 bytes
        const unsigned char* box = slot + (kb >> 3) * DF_BOX_BYTES + (kb & 7) * 64 + 16 * cx.t;
        const uint4 w_lo = *reinterpret_cast<const uint4*>(box + cx.g * (DF_BOX_COLS * 2));
        const uint4 w_hi = *reinterpret_cast<const uint4*>(box + (cx.g + 8) * (DF_BOX_COLS * 2));
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            const uint4 xf = *reinterpret_cast<const uint4*>(cx.xs + (size_t)(8 * mb + cx.g) * cx.x_pitch + col0 +
                                                            32 * kb + 8 * cx.t);
            mma_bf16(acc[mb], w_lo.x, w_hi.x, w_lo.y, w_hi.y, xf.x, xf.y);
            mma_bf16(acc[mb], w_lo.z, w_hi.z, w_lo.w, w_hi.w, xf.z, xf.w);
        }
    }
}

// What the epilogue of a unit needs from global memory, fetched before the unit's chunks are
// multiplied so that the round trip to L2 is hidden: thread tid owns element (feature row r,
// batch row m) of the unit, or (pair i, row m) of a rotated unit.
struct UnitInputs {
    float bias0, bias1, residual, cos_v, sin_v;
};
template <int MB, int HD>
__device__ __forceinline__ UnitInputs prepare_unit(const MxDfParams& p, const Cx& cx, const Gemm& d, int u) {
    constexpr int ROWS = 8 * MB;
    UnitInputs in = {0.f, 0.f, 0.f, 1.f, 0.f};
    if (d.mode == MODE_QKV) {
        const int per_head = HD >> 4;
        const int head = u / per_head, j = u - head * per_head;
        if (head < p.n_heads + p.n_kv_heads) {
            const int i = cx.tid & 7, m = cx.tid >> 3;
            if (cx.tid < 8 * ROWS && m < p.rows) {
                const int d_lo = 8 * j + i;
                if (d.bias != nullptr) {
                    in.bias0 = d.bias[head * HD + d_lo];
                    in.bias1 = d.bias[head * HD + d_lo + HD / 2];
                }
                const float angle = (float)p.context_lens[m] * d.layer->inv_freq[d_lo];
                in.cos_v = cosf(angle);
                in.sin_v = sinf(angle);
            }
        } else if (d.bias != nullptr && cx.tid < 16 * ROWS) {
            in.bias0 = d.bias[head * HD + 16 * j + (cx.tid & 15)];
        }
        return in;
    }
    const int r = cx.tid & 15, m = cx.tid >> 4;
    const int f = 16 * u + r;
    if (cx.tid < 16 * ROWS && f < d.N && m < p.rows) {
        if (d.bias != nullptr) in.bias0 = d.bias[f];
        if (d.mode == MODE_RESIDUAL) in.residual = ld_cg(p.x + (size_t)m * p.hidden + f);
    }
    return in;
}

// The eight warps' sums of one unit, added in warp order, then the epilogue of the product.
template <int MB, int HD>
__device__ __forceinline__ void finish_unit(const MxDfParams& p, Cx& cx, const Gemm& d, int u, int u_first, float (&acc)[MB][4],
                            const UnitInputs& in) {
    constexpr int ROWS = 8 * MB;
    consumer_sync();                       // the readers of the unit before are done with `red`
    {
        float* mine = cx.red + (size_t)cx.warp * 16 * ROWS;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            *reinterpret_cast<float2*>(mine + cx.g * ROWS + 8 * mb + 2 * cx.t) = make_float2(acc[mb][0], acc[mb][1]);
            *reinterpret_cast<float2*>(mine + (cx.g + 8) * ROWS + 8 * mb + 2 * cx.t) = make_float2(acc[mb][2], acc[mb][3]);
        }
    }
    consumer_sync();
    auto total = [&](int r, int m) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < DF_WARPS; ++w) v += cx.red[((size_t)w * 16 + r) * ROWS + m];
        return v;
    };
    if (d.mode == MODE_QKV) {
        const MxDfLayer& L = *d.layer;
        const int per_head = HD >> 4;
        const int head = u / per_head, j = u - head * per_head;
        const long long n_slots = L.n_pages * p.page_size;
        const size_t head_stride = (size_t)p.page_size * HD;
        const bool rotated = head < p.n_heads + p.n_kv_heads;
        const int m = rotated ? cx.tid >> 3 : cx.tid >> 4;
        if (cx.tid >= (rotated ? 8 : 16) * ROWS || m >= p.rows) return;
        long long page = 0;
        int offset = 0;
        if (head >= p.n_heads) {             // a key or value head: where the row's new token lives
            if (!L.writes_cache) return;
            const long long slot = p.slots[L.group][m];
            if (slot == -1) return;
            if (slot < 0 || slot >= n_slots) {
                atomicOr(cx.status, MX_STATUS_BAD_SLOT);
                return;
            }
            page = slot / p.page_size;
            offset = (int)(slot - page * p.page_size);
        }
        if (rotated) {
            const int i = cx.tid & 7;
            const int d_lo = 8 * j + i, d_hi = d_lo + HD / 2;
            // the separate kernels round the product to bfloat16 before rotating it: the same here
            const float lo = round_bf16(total(i, m) + in.bias0), hi = round_bf16(total(i + 8, m) + in.bias1);
            const __nv_bfloat16 r_lo = __float2bfloat16_rn(lo * in.cos_v - hi * in.sin_v);
            const __nv_bfloat16 r_hi = __float2bfloat16_rn(hi * in.cos_v + lo * in.sin_v);
            __nv_bfloat16* dst = head < p.n_heads
                                     ? p.q + (size_t)m * p.n_heads * HD + (size_t)head * HD
                                     : L.cache + ((size_t)page * 2 * p.n_kv_heads + (head - p.n_heads)) * head_stride +
                                           (size_t)offset * HD;
            dst[d_lo] = r_lo;
            dst[d_hi] = r_hi;
        } else {
            const int r = cx.tid & 15;
            const int vh = head - p.n_heads - p.n_kv_heads;
            L.cache[((size_t)page * 2 * p.n_kv_heads + p.n_kv_heads + vh) * head_stride +
                    (size_t)(16 * j + r) * p.page_size + offset] = __float2bfloat16_rn(total(r, m) + in.bias0);
        }
        return;
    }
    const int r = cx.tid & 15, m = cx.tid >> 4;
    const int f = 16 * u + r;
    if (cx.tid >= 16 * ROWS || f >= d.N || m >= p.rows) return;
    float v = total(r, m) + in.bias0;
    if (d.mode == MODE_RESIDUAL) {
        v += in.residual;
        p.x[(size_t)m * p.hidden + f] = v;
        p.xb[(size_t)m * p.hidden + f] = __float2bfloat16_rn(v);
        cx.stat_vals[m * DF_STAT_COLS + 16 * (u - u_first) + r] = v;
    } else if (d.mode == MODE_GELU) {
        p.mid[(size_t)m * p.inter + f] = __float2bfloat16_rn(gelu_tanh_fast(v));
    } else {
        p.logits[(size_t)m * p.vocab + f] = v;
    }
}

template <int MB, int HD>
__device__ __forceinline__ void consume_gemm(const MxDfParams& p, Cx& cx, const Gemm& d) {
    const int n_units = (d.N + 15) >> 4;
    const int u0 = unit_begin(blockIdx.x, n_units, p.grid), u1 = unit_begin(blockIdx.x + 1, n_units, p.grid);
    const int n_slices = (d.K + cx.x_cols - 1) / cx.x_cols;
    const int group_size = n_slices == 1 ? 1 : DF_UMAX;
    if (d.ln_w != nullptr) {
        DF_TIME(PF_COMBINE, cx.tid == 0);
        combine_stats(p, cx, d.ln_eps);
    }
    int staged = -1;
    for (int ug = u0; ug < u1; ug += group_size) {
        const int gn = min(group_size, u1 - ug);
        float acc[DF_UMAX][MB][4];
        UnitInputs inputs[DF_UMAX];
#pragma unroll
        for (int ul = 0; ul < DF_UMAX; ++ul) {
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) acc[ul][mb][0] = acc[ul][mb][1] = acc[ul][mb][2] = acc[ul][mb][3] = 0.f;
            if (ul < gn) inputs[ul] = prepare_unit<MB, HD>(p, cx, d, ug + ul);
        }
        for (int s = 0; s < n_slices; ++s) {
            const int k_begin = s * cx.x_cols, k_end = min(d.K, k_begin + cx.x_cols);
            if (staged != s) {
                DF_TIME(PF_STAGE, cx.tid == 0);
                stage_activations<MB>(p, cx, d, k_begin, k_end);
                staged = s;
            }
            DF_TIME(PF_CHUNKS, cx.tid == 0);
#pragma unroll
            for (int ul = 0; ul < DF_UMAX; ++ul) {
                if (ul < gn) {
                    for (int k0 = k_begin; k0 < k_end; k0 += DF_KC) {
                        const int kc = min(DF_KC, k_end - k0);
                        wait_full(cx);
#if !defined(DF_VARIANT) || DF_VARIANT != 1
                        multiply_chunk<MB>(cx, k0 - k_begin, kc >> 5, acc[ul]);
#endif
                        release_slot(cx);
                        ring_advance(cx);
                    }
                }
            }
        }
#pragma unroll
        for (int ul = 0; ul < DF_UMAX; ++ul)
            if (ul < gn) {
                DF_TIME(PF_FINISH, cx.tid == 0);
                finish_unit<MB, HD>(p, cx, d, ug + ul, u0, acc[ul], inputs[ul]);
            }
    }
    if (d.mode == MODE_RESIDUAL) write_partial_stats(p, cx, min(d.N, 16 * u1) - min(d.N, 16 * u0));
}

// ------------------------------------------------------------------ consumers: attention
template <int HD>
__device__ __forceinline__ void consume_attention(const MxDfParams& p, Cx& cx, const MxDfLayer& L) {
    constexpr int KB = HD / 32, NB = HD / 8;
    const int group = p.n_heads / p.n_kv_heads;
    const int shift = p.page_size == 8 ? 3 : (p.page_size == 16 ? 4 : 5);
    const int n_items = p.rows * p.n_kv_heads * p.n_splits;
    const int g = cx.g, t = cx.t;
    for (int item = blockIdx.x; item < n_items; item += p.grid) {
        const AttnItem a = attn_item(p, L, item);
        // rows of the MMA tile: the heads of the group, all at position ctx
        bool r_valid[2];
        uint4 qf[2][KB];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = g + 8 * i;
            r_valid[i] = r < group && a.seq >= 0;
            const __nv_bfloat16* qrow = p.q + (size_t)a.row * p.n_heads * HD + (size_t)(a.kh * group + min(r, group - 1)) * HD;
#pragma unroll
            for (int b = 0; b < KB; ++b)
                qf[i][b] = r_valid[i] ? ld_cg_u4(qrow + 32 * b + 8 * t) : make_uint4(0u, 0u, 0u, 0u);
        }
        float o[NB][4];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

        for (int ci = a.c_begin; ci < a.c_end; ++ci) {
            wait_full(cx);
            if (((ci - a.c_begin) & (DF_WARPS - 1)) == cx.warp && !*cx.abort_flag) {
                const int c0 = ci * DF_CHUNK;
                const __nv_bfloat16* ks = reinterpret_cast<const __nv_bfloat16*>(cx.ring + (size_t)cx.slot * DF_SLOT_BYTES);
                const __nv_bfloat16* vs = ks + DF_CHUNK * HD;
                // scores: block b gives this thread keys 8t + 2b, 8t + 2b + 1 of the chunk
                float s[4][4];
#pragma unroll
                for (int b = 0; b < 4; ++b) s[b][0] = s[b][1] = s[b][2] = s[b][3] = 0.f;
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
                    const __nv_bfloat16* kcol = ks + (size_t)(8 * (g >> 1) + (g & 1)) * HD + 8 * t + 32 * kb;
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        const uint4 kf = *reinterpret_cast<const uint4*>(kcol + 2 * b * HD);
                        mma_bf16(s[b], qf[0][kb].x, qf[1][kb].x, qf[0][kb].y, qf[1][kb].y, kf.x, kf.y);
                        mma_bf16(s[b], qf[0][kb].z, qf[1][kb].z, qf[0][kb].w, qf[1][kb].w, kf.z, kf.w);
                    }
                }
                const bool plain = c0 >= a.lo && c0 + DF_CHUNK - 1 <= a.ctx;
                float raw_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int b = 0; b < 4; ++b)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (!plain) {
                            const int key = c0 + 8 * t + 2 * b + (e & 1);
                            if (key > a.ctx || key < a.lo) s[b][e] = -INFINITY;
                        }
                        raw_max[e >> 1] = fmaxf(raw_max[e >> 1], s[b][e]);
                    }
                float m_new[2], alpha[2], m_use[2], sum[2] = {0.f, 0.f};
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    m_new[i] = fmaxf(m_run[i], raw_max[i] * L.scale_log2);
                    m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
                    m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
                    m_use[i] = (m_new[i] == -INFINITY) ? 0.f : m_new[i];
                    alpha[i] = fast_exp2(m_run[i] - m_use[i]);
                }
#pragma unroll
                for (int b = 0; b < 4; ++b)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float pv = fast_exp2(fmaf(s[b][e], L.scale_log2, -m_use[e >> 1]));
                        s[b][e] = pv;
                        sum[e >> 1] += pv;
                    }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
                    sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
                    l_run[i] = l_run[i] * alpha[i] + sum[i];
                    m_run[i] = m_new[i];
                }
                unsigned pa[2][4];
#pragma unroll
                for (int st = 0; st < 2; ++st) {
                    pa[st][0] = pack_bf16(s[2 * st][0], s[2 * st][1]);
                    pa[st][1] = pack_bf16(s[2 * st][2], s[2 * st][3]);
                    pa[st][2] = pack_bf16(s[2 * st + 1][0], s[2 * st + 1][1]);
                    pa[st][3] = pack_bf16(s[2 * st + 1][2], s[2 * st + 1][3]);
                }
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    o[nb][0] *= alpha[0]; o[nb][1] *= alpha[0];
                    o[nb][2] *= alpha[1]; o[nb][3] *= alpha[1];
                }
                // values [dim][slot] page by page; slots beyond the newest key hold no data yet
                const int in_chunk = 8 * t;
                const int pg = in_chunk >> shift, off = in_chunk & (p.page_size - 1);
                const size_t voff = (size_t)pg * p.page_size * HD + (size_t)g * p.page_size + off;
                unsigned keep[4];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int key = c0 + 8 * t + 2 * w;
                    keep[w] = (key <= a.ctx ? 0x0000ffffu : 0u) | (key + 1 <= a.ctx ? 0xffff0000u : 0u);
                }
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    uint4 vf = *reinterpret_cast<const uint4*>(vs + voff + (size_t)(8 * nb) * p.page_size);
                    vf.x &= keep[0]; vf.y &= keep[1]; vf.z &= keep[2]; vf.w &= keep[3];
                    mma_bf16(o[nb], pa[0][0], pa[0][1], pa[0][2], pa[0][3], vf.x, vf.y);
                    mma_bf16(o[nb], pa[1][0], pa[1][1], pa[1][2], pa[1][3], vf.z, vf.w);
                }
            }
            release_slot(cx);
            ring_advance(cx);
        }

        // ---- the eight warps' partial results, combined in the activation stage (free in this phase)
        float* buf_o = reinterpret_cast<float*>(cx.xs);           // [4][16][HD]
        float* buf_l = buf_o + 4 * 16 * HD;                       // [4][16]
        float* buf_m = buf_l + 4 * 16;                            // [8][16]
        consumer_sync();
        if (t == 0) {
            buf_m[cx.warp * 16 + g] = m_run[0];
            buf_m[cx.warp * 16 + g + 8] = m_run[1];
        }
        consumer_sync();
        float m_all[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < DF_WARPS; ++w) m = fmaxf(m, buf_m[w * 16 + g + 8 * i]);
            m_all[i] = m;
            const float wgt = (m_run[i] == -INFINITY) ? 0.f : fast_exp2(m_run[i] - m);
            l_run[i] *= wgt;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                o[nb][2 * i] *= wgt;
                o[nb][2 * i + 1] *= wgt;
            }
        }
        const int lanes4 = cx.warp & 3;
        if (cx.warp < 4) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float* dst = buf_o + ((size_t)lanes4 * 16 + g + 8 * i) * HD;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
                    *reinterpret_cast<float2*>(dst + 8 * nb + 2 * t) = make_float2(o[nb][2 * i], o[nb][2 * i + 1]);
                if (t == 0) buf_l[lanes4 * 16 + g + 8 * i] = l_run[i];
            }
        }
        consumer_sync();
        if (cx.warp >= 4) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float* dst = buf_o + ((size_t)lanes4 * 16 + g + 8 * i) * HD;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    float2 v = *reinterpret_cast<float2*>(dst + 8 * nb + 2 * t);
                    v.x += o[nb][2 * i];
                    v.y += o[nb][2 * i + 1];
                    *reinterpret_cast<float2*>(dst + 8 * nb + 2 * t) = v;
                }
                if (t == 0) buf_l[lanes4 * 16 + g + 8 * i] += l_run[i];
            }
        }
        // every thread of a quad holds the same m_all: thread t == 0 of warp 0 publishes it
        if (cx.warp == 0 && t == 0) {
            buf_m[g] = m_all[0];          // warp 0's own entries were read by everyone before the sync above
            buf_m[g + 8] = m_all[1];
        }
        consumer_sync();
        const int rows_here = a.seq >= 0 ? min(group, 16) : 0;
        for (int idx = cx.tid; idx < group * HD; idx += DF_CONSUMERS) {
            const int r = idx / HD, dcol = idx - r * HD;
            float acc = 0.f, l = 0.f;
            if (r < rows_here) {
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    acc += buf_o[((size_t)w * 16 + r) * HD + dcol];
                    l += buf_l[w * 16 + r];
                }
            }
            const int head = a.kh * group + r;
            if (p.n_splits == 1) {
                p.attn[(size_t)a.row * p.n_heads * HD + (size_t)head * HD + dcol] =
                    __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
            } else {
                const size_t base = ((size_t)a.row * p.n_heads + head) * p.n_splits + a.split;
                p.part_o[base * HD + dcol] = acc;
                if (dcol == 0) {
                    p.part_ml[base * 2] = r < rows_here ? buf_m[r] : -INFINITY;
                    p.part_ml[base * 2 + 1] = l;
                }
            }
        }
        consumer_sync();                  // the stage is reused by the next item or phase
    }
}

// The splits of every (row, head), merged by one warp each.
template <int HD>
__device__ __forceinline__ void merge_splits(const MxDfParams& p, Cx& cx) {
    constexpr int PER = HD / 32;
    const int n_items = p.rows * p.n_heads;
    for (int item = blockIdx.x * DF_WARPS + cx.warp; item < n_items; item += p.grid * DF_WARPS) {
        const size_t base = (size_t)item * p.n_splits;
        float m = -INFINITY;
        for (int s = 0; s < p.n_splits; ++s) m = fmaxf(m, ld_cg(p.part_ml + (base + s) * 2));
        float l = 0.f, acc[PER];
#pragma unroll
        for (int e = 0; e < PER; ++e) acc[e] = 0.f;
        for (int s = 0; s < p.n_splits; ++s) {
            const float2 ml = ld_cg2(p.part_ml + (base + s) * 2);
            if (ml.x == -INFINITY) continue;
            const float wgt = exp2f(ml.x - m);
            l += ml.y * wgt;
            const float* po = p.part_o + (base + s) * HD + PER * cx.lane;
            if (PER == 4) {
                const float4 v = ld_cg4(po);
                acc[0] += v.x * wgt; acc[1] += v.y * wgt; acc[2] += v.z * wgt; acc[3] += v.w * wgt;
            } else {
                const float2 v = ld_cg2(po);
                acc[0] += v.x * wgt; acc[1] += v.y * wgt;
            }
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = p.attn + (size_t)item * HD + PER * cx.lane;
#pragma unroll
        for (int e = 0; e < PER; e += 2)
            *reinterpret_cast<unsigned*>(dst + e) = pack_bf16(acc[e] * inv, acc[e + 1] * inv);
    }
}

// Row m of the residual stream starts as the embedding of its token.
__device__ __forceinline__ void embed_rows(const MxDfParams& p, Cx& cx) {
    const int f0 = unit_begin(blockIdx.x, p.hidden, p.grid), f1 = unit_begin(blockIdx.x + 1, p.hidden, p.grid);
    const int count = f1 - f0;
    for (int idx = cx.tid; idx < p.rows * count; idx += DF_CONSUMERS) {
        const int m = idx / count, i = idx - m * count;
        int token = p.token_ids[m];
        if (token < 0 || token >= p.vocab) {
            atomicOr(cx.status, MX_STATUS_BAD_TOKEN_ID);
            token = 0;
        }
        const float v = __bfloat162float(p.embedding[(size_t)token * p.hidden + f0 + i]);
        p.x[(size_t)m * p.hidden + f0 + i] = v;
        p.xb[(size_t)m * p.hidden + f0 + i] = p.embedding[(size_t)token * p.hidden + f0 + i];
        cx.stat_vals[m * DF_STAT_COLS + i] = v;
    }
    write_partial_stats(p, cx, count);
}

// ------------------------------------------------------------------ the kernel
__device__ __forceinline__ Gemm qkv_gemm(const MxDfParams& p, const MxDfLayer& L) {
    Gemm d = {};
    d.map = L.qkv_map; d.W = L.qkv_w; d.bias = L.qkv_b; d.N = (p.n_heads + 2 * p.n_kv_heads) * p.head_dim; d.K = p.hidden;
    d.mode = MODE_QKV; d.ln_w = L.ln1_w; d.ln_b = L.ln1_b; d.ln_eps = L.ln1_eps; d.layer = &L;
    return d;
}
__device__ __forceinline__ Gemm o_gemm(const MxDfParams& p, const MxDfLayer& L) {
    Gemm d = {};
    d.map = L.o_map; d.W = L.o_w; d.bias = L.o_b; d.N = p.hidden; d.K = p.n_heads * p.head_dim; d.mode = MODE_RESIDUAL;
    d.src = p.attn; d.src_ld = p.n_heads * p.head_dim;
    return d;
}
__device__ __forceinline__ Gemm fc_gemm(const MxDfParams& p, const MxDfLayer& L) {
    Gemm d = {};
    d.map = L.fc_map; d.W = L.fc_w; d.bias = L.fc_b; d.N = p.inter; d.K = p.hidden; d.mode = MODE_GELU;
    d.ln_w = L.ln2_w; d.ln_b = L.ln2_b; d.ln_eps = L.ln2_eps;
    return d;
}
__device__ __forceinline__ Gemm proj_gemm(const MxDfParams& p, const MxDfLayer& L) {
    Gemm d = {};
    d.map = L.proj_map; d.W = L.proj_w; d.bias = L.proj_b; d.N = p.hidden; d.K = p.inter; d.mode = MODE_RESIDUAL;
    d.src = p.mid; d.src_ld = p.inter;
    return d;
}
__device__ __forceinline__ Gemm layer_gemm(const MxDfParams& p, const MxDfLayer& L, int which) {
    if (which == 0) return qkv_gemm(p, L);
    if (which == 1) return o_gemm(p, L);
    if (which == 2) return fc_gemm(p, L);
    return proj_gemm(p, L);
}
__device__ __forceinline__ Gemm head_gemm(const MxDfParams& p) {
    Gemm d = {};
    d.map = p.head_map; d.W = p.head; d.N = p.vocab; d.K = p.hidden; d.mode = MODE_LOGITS;
    d.ln_w = p.final_w; d.ln_b = p.final_b; d.ln_eps = p.final_eps;
    return d;
}

template <int HD, int MB>
__global__ void __launch_bounds__(DF_THREADS, 1) decode_fused_kernel(const __grid_constant__ MxDfParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int abort_flag;
    Cx cx;
    cx.ring = smem;
    cx.xs = reinterpret_cast<__nv_bfloat16*>(smem + (size_t)p.ring_slots * DF_SLOT_BYTES);
    cx.red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(cx.xs) + p.xs_bytes);
    cx.stat_vals = cx.red + DF_WARPS * 16 * 8 * MB;
    cx.row_stats = cx.stat_vals + 8 * MB * DF_STAT_COLS;
    cx.full = reinterpret_cast<unsigned long long*>(cx.row_stats + 32);
    cx.empty = cx.full + p.ring_slots;
    cx.xs_bar = cx.empty + p.ring_slots;
    cx.xs_phase = 0;
    cx.abort_flag = &abort_flag;
    cx.status = p.status;
    cx.slots = p.ring_slots;
    cx.x_cols = p.x_cols;
    cx.x_pitch = p.x_cols + 32;
    cx.slot = 0;
    cx.round = 0;
    cx.epoch = 0;
    cx.tid = threadIdx.x;
    cx.warp = threadIdx.x >> 5;
    cx.lane = threadIdx.x & 31;
    cx.g = cx.lane >> 2;
    cx.t = cx.lane & 3;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.ring_slots; ++s) {
            mbar_init(&cx.full[s], 1);
            mbar_init(&cx.empty[s], DF_WARPS);
        }
        mbar_init(cx.xs_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    const bool merged = p.n_splits > 1;
    const unsigned per_layer = merged ? 6u : 5u;

    DF_TIME(PF_TOTAL, cx.tid == 0);
    cx.pid = cx.warp - DF_WARPS;
    cx.seq = 0;
#ifdef DF_PROFILE
    cx.t_wait_full = cx.t_wait_empty = 0;
#endif
    if (cx.warp >= DF_WARPS) {
        // ================= producer warp
        DF_TIME(PF_PRODUCER_TOTAL, cx.lane == 0);
        // products 0..3 of every layer (QKV, output, up, down), then the head: one call site each,
        // so that the block's state stays in registers
        for (int l = 0; l <= p.n_layers; ++l) {
            const bool last = l == p.n_layers;
            const MxDfLayer& L = p.layers[last ? 0 : l];
            for (int which = 0; which < (last ? 1 : 4); ++which) {
                produce_gemm(p, cx, last ? head_gemm(p) : layer_gemm(p, L, which));
                if (!last && which == 0)
                    produce_attention<HD>(p, cx, L, 2u + (unsigned)l * per_layer);   // barrier after this layer's QKV
            }
        }
#ifdef DF_PROFILE
        if (cx.lane == 0) atomicAdd(&g_profile[blockIdx.x][PF_WAIT_EMPTY], (unsigned long long)cx.t_wait_empty);
#endif
        if (*cx.abort_flag) {
            // copies that were issued but will not be consumed: wait for them before the block ends
            for (int s = 0; s < p.ring_slots; ++s) {
                const bool issued = cx.round > 0 || s < cx.slot;
                if (!issued) continue;
                const unsigned parity = (s < cx.slot ? cx.round : cx.round - 1u) & 1u;
                for (unsigned spin = 0; spin < (1u << 20); ++spin)
                    if (mbar_try_wait(&cx.full[s], parity)) break;
            }
        }
        return;
    }

    // ================= consumer warps
    embed_rows(p, cx);
    grid_barrier(p, cx);                                        // 1
    for (int l = 0; l <= p.n_layers; ++l) {
        const bool last = l == p.n_layers;
        const MxDfLayer& L = p.layers[last ? 0 : l];
        for (int which = 0; which < (last ? 1 : 4); ++which) {
            consume_gemm<MB, HD>(p, cx, last ? head_gemm(p) : layer_gemm(p, L, which));
            if (last) break;
            if (which == 0) fence_async_proxy();     // the new keys and values are read by other blocks' bulk copies
            grid_barrier(p, cx);                         // after QKV: 2 + l * per_layer
            if (which == 0) {
                {
                    DF_TIME(PF_ATTENTION, cx.tid == 0);
                    consume_attention<HD>(p, cx, L);
                }
                grid_barrier(p, cx);
                if (merged) {
                    {
                        DF_TIME(PF_MERGE, cx.tid == 0);
                        merge_splits<HD>(p, cx);
                    }
                    grid_barrier(p, cx);
                }
            }
        }
    }
#ifdef DF_PROFILE
    if (cx.tid == 0) g_profile[blockIdx.x][PF_WAIT_CHUNK] += (unsigned long long)cx.t_wait_full;
#endif
}

size_t fixed_smem_bytes(int mb, int ring_slots) {
    return (size_t)DF_WARPS * 16 * 8 * mb * 4 + (size_t)8 * mb * DF_STAT_COLS * 4 + 32 * 4 + (size_t)(2 * ring_slots + 2) * 8;
}

template <int HD, int MB>
int launch_fused(const MxDfParams& p, size_t smem, cudaStream_t stream) {
    auto kernel = decode_fused_kernel<HD, MB>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) MX_REFUSE("fused decode: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, DF_THREADS, smem);
    if (e != cudaSuccess || per_sm < 1) MX_REFUSE("fused decode: a block does not fit an SM (%zu bytes of shared memory)", smem);
    e = cudaMemsetAsync(p.barrier, 0, sizeof(unsigned), stream);
    if (e != cudaSuccess) MX_REFUSE("fused decode: cannot reset the barrier: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(p.grid);
    config.blockDim = dim3(DF_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeCooperative;      // all blocks resident: they wait on one another
    attribute[0].val.cooperative = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    e = cudaLaunchKernelEx(&config, kernel, p);
    if (e != cudaSuccess) {
        mx_set_error("fused decode: launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return MX_OK;
}

}  // namespace

#ifdef DF_PROFILE
extern "C" int mx_decode_fused_profile(unsigned long long* out, int reset) {
    cudaDeviceSynchronize();
    if (out) cudaMemcpyFromSymbol(out, g_profile, sizeof(unsigned long long) * 256 * PF_COUNT);
    if (reset) {
        static unsigned long long zeros[256 * PF_COUNT];
        cudaMemcpyToSymbol(g_profile, zeros, sizeof(zeros));
    }
    return MX_OK;
}
#endif

typedef CUresult (*DfEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Writes the 128-byte tensor map of a [rows][cols] bfloat16 matrix (rows contiguous) with boxes of
// 256 columns by `box_rows` rows to `out` (host memory); the caller copies it to the device.
extern "C" int mx_decode_fused_weight_map(void* out, const void* weight, long long rows, long long cols,
                                          int box_rows) {
    static DfEncodeTiledFn encode = nullptr;
    if (encode == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) == cudaSuccess &&
            query == cudaDriverEntryPointSuccess)
            encode = reinterpret_cast<DfEncodeTiledFn>(ptr);
    }
    if (encode == nullptr) MX_REFUSE("fused decode: the driver does not offer cuTensorMapEncodeTiled");
    if (cols % 8 != 0 || reinterpret_cast<uintptr_t>(weight) % 16 != 0)
        MX_REFUSE("fused decode: a weight matrix needs 16-byte aligned rows (%lld columns)", cols);
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)DF_BOX_COLS, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap map;
    const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(weight), dims, strides,
                               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) MX_REFUSE("fused decode: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    memcpy(out, &map, sizeof(map));
    return MX_OK;
}

extern "C" int mx_decode_fused_sizes(int* layer_bytes, int* params_bytes) {
    *layer_bytes = (int)sizeof(MxDfLayer);
    *params_bytes = (int)sizeof(MxDfParams);
    return MX_OK;
}

// Chooses the shared-memory split (activation stage, ring) for a model and says whether the
// kernel takes it: fills x_cols, xs_bytes, ring_slots and grid of `p`. Returns MX_OK or refuses.
extern "C" int mx_decode_fused_plan(MxDfParams* p) {
    if (p->rows < 1 || p->rows > 16) MX_REFUSE("fused decode takes 1 to 16 rows, not %d", p->rows);
    if (p->head_dim != 64 && p->head_dim != 128) MX_REFUSE("fused decode is built for head_dim 64 and 128, not %d", p->head_dim);
    if (p->page_size != 8 && p->page_size != 16 && p->page_size != 32)
        MX_REFUSE("fused decode takes pages of 8, 16 or 32 slots, not %d", p->page_size);
    if (p->n_kv_heads < 1 || p->n_heads % p->n_kv_heads != 0 || p->n_heads / p->n_kv_heads > 16)
        MX_REFUSE("fused decode takes query groups of at most 16 heads (%d heads, %d kv heads)", p->n_heads, p->n_kv_heads);
    if (p->hidden % 32 != 0 || p->inter % 32 != 0)
        MX_REFUSE("fused decode needs hidden and intermediate sizes that are multiples of 32 (%d, %d)", p->hidden, p->inter);
    int device = 0, sms = 0, smem_max = 0, cooperative = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device);
    if (!cooperative) MX_REFUSE("fused decode needs cooperative launches");
    p->grid = sms;
    const int mb = p->rows <= 8 ? 1 : 2;
    if ((p->hidden + sms - 1) / sms + 1 > DF_STAT_COLS || 16 * (((p->hidden + 15) / 16 + sms - 1) / sms + 1) > DF_STAT_COLS)
        MX_REFUSE("fused decode: hidden size %d is too wide for %d blocks", p->hidden, sms);
    const int k_max = p->hidden > p->n_heads * p->head_dim ? p->hidden : p->n_heads * p->head_dim;
    // the stage holds whole rows of the narrowest products; wider ones (the down product) go in slices
    int x_cols = ((k_max + DF_KC - 1) / DF_KC) * DF_KC;
    const int x_cap = (mb == 1 ? 4096 : 3072);
    if (x_cols > x_cap) x_cols = x_cap;
    p->x_cols = x_cols;
    size_t xs = (size_t)8 * mb * (x_cols * 2 + 64);
    const size_t merge = (size_t)4 * 16 * p->head_dim * 4 + 4 * 16 * 4 + 8 * 16 * 4;
    if (xs < merge) xs = merge;
    xs = (xs + 127) & ~(size_t)127;
    p->xs_bytes = (int)xs;
    const long long budget = (long long)smem_max - 64;      // the kernel's one static word
    int slots = 0;
    while (slots < 14 && (long long)(slots + 1) * DF_SLOT_BYTES + (long long)xs + (long long)fixed_smem_bytes(mb, slots + 1) <= budget)
        ++slots;
    if (slots < 3) MX_REFUSE("fused decode: only %d ring slots fit beside a %zu-byte activation stage", slots, xs);
    p->ring_slots = slots;
    return MX_OK;
}

extern "C" int mx_decode_fused(const MxDfParams* params, cudaStream_t stream) {
    MxDfParams p = *params;
    MxDfParams check = p;
    const int rc = mx_decode_fused_plan(&check);
    if (rc != MX_OK) return rc;
    if (check.grid != p.grid || check.x_cols != p.x_cols || check.xs_bytes != p.xs_bytes || check.ring_slots != p.ring_slots)
        MX_REFUSE("fused decode: the plan in the argument block does not match this device");
    if (p.n_splits < 1) MX_REFUSE("fused decode: n_splits %d", p.n_splits);
    const int mb = p.rows <= 8 ? 1 : 2;
    const size_t smem = (size_t)p.ring_slots * DF_SLOT_BYTES + (size_t)p.xs_bytes + fixed_smem_bytes(mb, p.ring_slots);
    if (p.head_dim == 64) return mb == 1 ? launch_fused<64, 1>(p, smem, stream) : launch_fused<64, 2>(p, smem, stream);
    return mb == 1 ? launch_fused<128, 1>(p, smem, stream) : launch_fused<128, 2>(p, smem, stream);
}
