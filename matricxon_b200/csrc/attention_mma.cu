// Tensor-core paged attention for bfloat16: prompt portions and decode tokens.
//
// Same mathematics and visibility rule as attention.cu (query at p sees key j iff j <= p and
// (window == 0 or j > p - window); scores q.k * scale; float softmax; query head h reads KV
// head h / group), cf. app/native/src/mx_attention.c:16-68 and
// app/architectures/qwen_layers.py:12-17,94-100.
//
// Rows. For one sequence and one KV head the query rows are the pairs (token, head in
// group), token-major: row r = t * group + h. A warp owns 16 consecutive rows (an MMA M
// tile); with grouped queries those rows sit on one or two tokens, so they share nearly the
// same causal limit and every key they load is used by all of them.
//
// Work. A block (four warps for wide tiles, eight for narrow ones) owns a tile of rows of one (sequence, KV head) and a split of
// the keys, walked in chunks of 32 absolute positions. A page's keys for one KV head are one
// contiguous piece of memory and so are its values, so a chunk reaches shared memory as a
// few bulk asynchronous copies (cp.async.bulk, completion counted on an mbarrier) issued by
// one thread, several chunks ahead of the arithmetic. Pages must hold 8, 16 or 32 slots.
//   * "wide" tiles (64 rows, prompt portions): each warp has 16 rows of its own and every
//     warp works on every chunk, two chunks per softmax update, so a chunk is fetched once
//     for 64 rows (four stages a block);
//   * "narrow" tiles (at most 16 rows, decode tokens): all eight warps hold the same rows,
//     each streams every eighth chunk through a stage of its own (its block-table entries read
//     ahead into shared memory), and their partial results are combined in shared memory
//     (each warp's weight per row computed once, then float4 sums). A warp's first chunk, if
//     all its keys were cached by earlier steps, is asked for before the kernel waits for its
//     predecessor in the stream (the one that computes the queries and this step's keys).
// Every wait on an mbarrier is bounded: after SPIN_LIMIT polls the kernel sets
// MX_STATUS_WAIT_TIMEOUT in the step's status word and goes on, so it always ends.
// Per chunk and warp: S = Q K^T with mma.sync.m16n8k16 (bf16 in, float out), float online
// softmax in registers, O += P V. Two orderings are chosen so that every fragment is 16
// contiguous bytes: the contraction over head dims runs in a permuted order (thread t of a
// quad takes dims 8t..8t+7 of each block of 32), and the 8 score columns of an MMA are
// assigned to keys so that thread t ends up holding the scores of keys 8t..8t+7 of the
// chunk, which is the A fragment of P V against values stored [dim][key].
// With more than one split a block writes unnormalised partials (max, sum, values) in the
// layout of attention.cu, and that file's merge kernel combines them.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int MMA_WARPS = 4;        // wide tiles: 16 rows each
constexpr int MMA_THREADS = MMA_WARPS * 32;
constexpr int NARROW_WARPS = 8;     // narrow tiles: all warps hold the same rows and share the chunks
constexpr int NARROW_THREADS = NARROW_WARPS * 32;
constexpr int CHUNK = 32;
constexpr int WIDE_STAGES = 4;      // chunks in flight per block (two pairs), wide tiles
constexpr int NARROW_STAGES = 1;    // chunks in flight per warp, narrow tiles
constexpr int NARROW_TABLE = 512;   // block-table entries a narrow tile's block reads ahead (8,192 positions in pages of 16)
constexpr int SPIN_LIMIT = 1 << 22;

struct MmaAttnParams {
    const __nv_bfloat16* q;      // [tokens][q_stride], head h at h * HD
    const __nv_bfloat16* cache;  // [page][2][kv head][page_size * HD]: K [slot][dim], V [dim][slot]
    __nv_bfloat16* out;          // [tokens][out_stride]
    float* part_o;               // [tokens][heads][splits][HD]
    float* part_ml;              // [tokens][heads][splits][2]
    const int* block_tables;     // [seqs][bt_stride]
    const int* cu_q;             // [seqs + 1] first token row of each sequence
    const int* context_lens;     // [seqs] tokens cached before this step
    const int* tiles;            // [n_tiles][2]: (sequence, first row of the tile)
    int* status;
    long long n_pages;
    int n_tiles, q_stride, out_stride, bt_stride;
    int n_heads, n_kv_heads, page_size, page_shift, window, n_splits;
    float scale_log2;            // scale * log2(e)
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2,
                                         unsigned a3, unsigned b0, unsigned b1) {
    // not volatile: a pure function of its operands, which the compiler may schedule among the loads
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
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

// ---- mbarrier + bulk copy (all waits bounded)
__device__ __forceinline__ unsigned smem_addr(const void* ptr) {
    return (unsigned)__cvta_generic_to_shared(ptr);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
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
__device__ __forceinline__ void mbar_wait(unsigned long long* bar, unsigned parity, int* status) {
    for (int spin = 0; spin < SPIN_LIMIT; ++spin)
        if (mbar_try_wait(bar, parity)) return;
    atomicOr(status, MX_STATUS_WAIT_TIMEOUT);       // give up: the results are void, the kernel ends
}
__device__ __forceinline__ void bulk_copy(void* smem_dst, const void* gmem_src, unsigned bytes,
                                          unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
            smem_addr(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}

// Brings the chunk starting at key c0 into a stage: keys as [key][HD], values page by page as
// [HD][page_size]. `who` of `n_who` cooperating threads; thread 0 issues the copies. Pages the
// request no longer holds (they lie wholly outside [lo, hi]) are filled with zeros instead.
template <int HD>
__device__ __forceinline__ void issue_chunk(const MmaAttnParams& p, __nv_bfloat16* ks,
                                            __nv_bfloat16* vs, unsigned long long* bar, int c0, int lo,
                                            int hi, const int* bt, const __nv_bfloat16* kbase,
                                            const __nv_bfloat16* vbase, size_t page_stride, int who,
                                            int n_who, const int* cached = nullptr) {
    const int ps = p.page_size;
    const int pages = CHUNK >> p.page_shift;
    const unsigned tile_bytes = (unsigned)(ps * HD * sizeof(__nv_bfloat16));
    long long page_of[4];
    unsigned total = 0;
#pragma unroll
    for (int pg = 0; pg < 4; ++pg) {
        page_of[pg] = -1;
        if (pg < pages) {
            const int key0 = c0 + pg * ps;
            if (key0 <= hi && key0 + ps - 1 >= lo) {
                const int lp = key0 >> p.page_shift;
                // `cached`: this chunk's block-table entries, read ahead into shared memory
                const long long page = cached != nullptr ? cached[pg] : (lp < p.bt_stride ? bt[lp] : -1);
                if (page >= 0 && page < p.n_pages) {
                    page_of[pg] = page;
                    total += 2 * tile_bytes;
                } else if (who == 0) {
                    atomicOr(p.status, MX_STATUS_BAD_PAGE);
                }
            }
        }
    }
    if (who == 0) {
        mbar_expect_tx(bar, total);
#pragma unroll
        for (int pg = 0; pg < 4; ++pg)
            if (pg < pages && page_of[pg] >= 0) {
                bulk_copy(ks + (size_t)pg * ps * HD, kbase + (size_t)page_of[pg] * page_stride, tile_bytes, bar);
                bulk_copy(vs + (size_t)pg * ps * HD, vbase + (size_t)page_of[pg] * page_stride, tile_bytes, bar);
            }
    }
#pragma unroll
    for (int pg = 0; pg < 4; ++pg)
        if (pg < pages && page_of[pg] < 0) {
            uint4* kz = reinterpret_cast<uint4*>(ks + (size_t)pg * ps * HD);
            uint4* vz = reinterpret_cast<uint4*>(vs + (size_t)pg * ps * HD);
            for (int i = who; i < (int)(tile_bytes / 16); i += n_who) {
                kz[i] = make_uint4(0, 0, 0, 0);
                vz[i] = make_uint4(0, 0, 0, 0);
            }
        }
}

struct One { static constexpr int value = 1; };
struct Two { static constexpr int value = 2; };

template <int HD, bool NARROW>
__global__ void __launch_bounds__(NARROW ? NARROW_THREADS : MMA_THREADS, NARROW ? 1 : 3)
attention_mma_kernel(const MmaAttnParams p) {
    constexpr int KB = HD / 32;                 // 32-wide blocks of the head dim
    constexpr int NB = HD / 8;                  // 8-wide output column blocks
    constexpr int STAGE_ELEMS = 2 * CHUNK * HD; // keys then values
    constexpr int TILE_ROWS = NARROW ? 16 : 16 * MMA_WARPS;
    constexpr int N_STAGES = NARROW ? NARROW_STAGES * NARROW_WARPS : WIDE_STAGES;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* stages = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __shared__ __align__(8) unsigned long long bars[N_STAGES];
    __shared__ int narrow_table[NARROW ? NARROW_TABLE : 1];   // the sequence's first block-table entries

    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x, kh = blockIdx.y, split = blockIdx.z;
    // no tile list: tile i is the whole of sequence i (a batch of decoding requests), one look-up less
    const int seq = p.tiles ? p.tiles[2 * tile] : tile, tile_row0 = p.tiles ? p.tiles[2 * tile + 1] : 0;
    if (NARROW) {
        // the block-table row sets out together with the sequence's lengths (it does not depend on
        // them): one trip to memory instead of two before the first page can be asked for
        const int* row = p.block_tables + (size_t)seq * p.bt_stride;
        for (int e = threadIdx.x; e < min(p.bt_stride, NARROW_TABLE); e += blockDim.x) narrow_table[e] = row[e];
    }
    const int group = p.n_heads / p.n_kv_heads;
    const int q_start = p.cu_q[seq];
    const int q_len = p.cu_q[seq + 1] - q_start;
    const int ctx = p.context_lens[seq];
    const int n_rows = q_len * group;
    if (tile_row0 >= n_rows) return;            // a padding sequence of a fixed-size batch

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < N_STAGES; ++s) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    // rows of this block and of this warp
    const int tile_last = min(tile_row0 + TILE_ROWS - 1, n_rows - 1);
    const int row0 = NARROW ? tile_row0 : tile_row0 + 16 * warp;
    const bool warp_has_rows = row0 < n_rows;
    const int last_row = min(row0 + 15, n_rows - 1);

    int r_tok[2], r_head[2], r_pos[2], r_lo[2];
    bool r_valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = row0 + g + 8 * i;
        r_valid[i] = r < n_rows;
        const int rr = r_valid[i] ? r : tile_last;
        r_tok[i] = rr / group;
        r_head[i] = rr - r_tok[i] * group;
        r_pos[i] = ctx + r_tok[i];
        r_lo[i] = p.window > 0 ? max(0, r_pos[i] - p.window + 1) : 0;
    }
    // key range of the block (what is fetched) and of the warp (what it computes)
    const int hi_tile = ctx + tile_last / group;
    const int lo_tile = p.window > 0 ? max(0, ctx + tile_row0 / group - p.window + 1) : 0;
    const int hi_warp = warp_has_rows ? ctx + last_row / group : -1;
    const int lo_warp = p.window > 0 ? max(0, ctx + row0 / group - p.window + 1) : 0;
    // rows of the warp see every key of a chunk that lies in [all_lo, all_hi]: no mask needed
    const int all_hi = warp_has_rows ? ctx + row0 / group : -1;
    const int all_lo = p.window > 0 ? max(0, hi_warp - p.window + 1) : 0;
    const bool rows_full = row0 + 15 < n_rows;
    const int first_chunk = lo_tile / CHUNK, last_chunk = hi_tile / CHUNK;
    const int n_chunks = last_chunk - first_chunk + 1;
    const int per_split = (n_chunks + p.n_splits - 1) / p.n_splits;
    const int c_begin = first_chunk + split * per_split;
    const int c_end = min(last_chunk + 1, c_begin + per_split);

    const int* bt = p.block_tables + (size_t)seq * p.bt_stride;
    const size_t head_stride = (size_t)p.page_size * HD;
    const size_t page_stride = 2 * (size_t)p.n_kv_heads * head_stride;
    const __nv_bfloat16* kbase = p.cache + (size_t)kh * head_stride;
    const __nv_bfloat16* vbase = p.cache + (size_t)(p.n_kv_heads + kh) * head_stride;
    // Narrow tiles: up to here only step metadata was read (uploaded before the step, written by no
    // kernel), and the keys and values of positions before this step are in the cache since earlier
    // steps. So this warp's first chunk, if it holds none of this step's positions, sets out now, under
    // the tail of the kernel that computes the queries and the newest keys.
    __nv_bfloat16* my_stages = stages + (size_t)(NARROW ? warp : 0) * NARROW_STAGES * STAGE_ELEMS;
    unsigned long long* my_bars = bars + (NARROW ? warp : 0) * NARROW_STAGES;
    const int my_first = c_begin + warp;
    const int my_count = NARROW && my_first < c_end ? (c_end - my_first + NARROW_WARPS - 1) / NARROW_WARPS : 0;
    // This warp's chunks find their pages in the row read ahead at the top (entries beyond what was
    // kept are looked up in global memory).
    auto cached_for = [&](int i) -> const int* {
        const int pages = CHUNK >> p.page_shift;
        const int first = (my_first + NARROW_WARPS * i) * pages;
        return first + pages <= min(p.bt_stride, NARROW_TABLE) ? narrow_table + first : nullptr;
    };
    const bool first_is_old = (my_first + 1) * CHUNK <= ctx;
    if (NARROW && my_count > 0 && first_is_old)
        issue_chunk<HD>(p, my_stages, my_stages + CHUNK * HD, &my_bars[0], my_first * CHUNK, lo_tile,
                        hi_tile, bt, kbase, vbase, page_stride, lane, 32, cached_for(0));
    // queries and the newest keys and values come from the kernels before this one
    pdl_wait();
    // Q fragments: 16 bytes of each owned row per 32-wide block. A row beyond the tile reads the
    // tile's last row (r_tok, r_head point there): its scores are masked and it is never written, and
    // a load that is not conditional is not waited for here.
    uint4 qf[2][KB];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const __nv_bfloat16* qrow = after_wait(p.q) + (size_t)(q_start + r_tok[i]) * p.q_stride +
                                    (size_t)(kh * group + r_head[i]) * HD;
#pragma unroll
        for (int b = 0; b < KB; ++b) qf[i][b] = *reinterpret_cast<const uint4*>(qrow + 32 * b + 8 * t);
    }

    float o[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    // ---- arithmetic on one chunk, or on two consecutive chunks with one softmax update for both
    auto compute = [&](auto n_chunks_tag, const __nv_bfloat16* ks0, const __nv_bfloat16* vs0,
                       const __nv_bfloat16* ks1, const __nv_bfloat16* vs1, int c0) {
        constexpr int NCH = decltype(n_chunks_tag)::value;
        const __nv_bfloat16* ksv[2] = {ks0, ks1};
        const __nv_bfloat16* vsv[2] = {vs0, vs1};
        // scores: block b of a chunk gives this thread that chunk's keys 8t + 2b, 8t + 2b + 1.
        // Column g of block b is key 8 (g / 2) + 2b + (g % 2). The 32-wide blocks of the head dim
        // are the outer loop, so consecutive MMAs go to different accumulators.
        float s[NCH][4][4];
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
            for (int b = 0; b < 4; ++b) s[ch][b][0] = s[ch][b][1] = s[ch][b][2] = s[ch][b][3] = 0.f;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
            for (int ch = 0; ch < NCH; ++ch) {
                const __nv_bfloat16* kcol = ksv[ch] + (size_t)(8 * (g >> 1) + (g & 1)) * HD + 8 * t + 32 * kb;
                // the two MMAs into one accumulator depend on one another: four accumulators between them
                uint4 kf[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) kf[b] = *reinterpret_cast<const uint4*>(kcol + 2 * b * HD);
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    mma_bf16(s[ch][b], qf[0][kb].x, qf[1][kb].x, qf[0][kb].y, qf[1][kb].y, kf[b].x, kf[b].y);
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    mma_bf16(s[ch][b], qf[0][kb].z, qf[1][kb].z, qf[0][kb].w, qf[1][kb].w, kf[b].z, kf[b].w);
            }
        // mask (only where the chunks cross an edge), running max and sum for rows g, g + 8
        float m_new[2] = {m_run[0], m_run[1]};
        const bool plain = rows_full && c0 >= all_lo && c0 + NCH * CHUNK - 1 <= all_hi;
        // scores stay unscaled until the exponential: exp2(s * c - m * c) is one FMA and one ex2
        // (c > 0, so the maximum of s * c is c times the maximum of s)
        float raw_max[2] = {-INFINITY, -INFINITY};
        if (plain) {
#pragma unroll
            for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
                for (int b = 0; b < 4; ++b)
#pragma unroll
                    for (int e = 0; e < 4; ++e) raw_max[e >> 1] = fmaxf(raw_max[e >> 1], s[ch][b][e]);
        } else {
#pragma unroll
            for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
                for (int b = 0; b < 4; ++b)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = e >> 1;
                        const int key = c0 + CHUNK * ch + 8 * t + 2 * b + (e & 1);
                        const bool visible = r_valid[i] && key <= r_pos[i] && key >= r_lo[i];
                        s[ch][b][e] = visible ? s[ch][b][e] : -INFINITY;
                        raw_max[i] = fmaxf(raw_max[i], s[ch][b][e]);
                    }
        }
        m_new[0] = fmaxf(m_new[0], raw_max[0] * p.scale_log2);
        m_new[1] = fmaxf(m_new[1], raw_max[1] * p.scale_log2);
        float alpha[2], sum[2] = {0.f, 0.f}, m_use[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
            m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
            // a row with nothing visible so far keeps max = -inf; subtract 0 then, exp2(-inf) = 0
            m_use[i] = (m_new[i] == -INFINITY) ? 0.f : m_new[i];
            alpha[i] = fast_exp2(m_run[i] - m_use[i]);
        }
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
            for (int b = 0; b < 4; ++b)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = fast_exp2(fmaf(s[ch][b][e], p.scale_log2, -m_use[e >> 1]));
                    s[ch][b][e] = pv;
                    sum[e >> 1] += pv;
                }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
            sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
            l_run[i] = l_run[i] * alpha[i] + sum[i];
            m_run[i] = m_new[i];
        }
        unsigned pa[NCH][2][4];
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
            for (int st = 0; st < 2; ++st) {
                pa[ch][st][0] = pack_bf16(s[ch][2 * st][0], s[ch][2 * st][1]);
                pa[ch][st][1] = pack_bf16(s[ch][2 * st][2], s[ch][2 * st][3]);
                pa[ch][st][2] = pack_bf16(s[ch][2 * st + 1][0], s[ch][2 * st + 1][1]);
                pa[ch][st][3] = pack_bf16(s[ch][2 * st + 1][2], s[ch][2 * st + 1][3]);
            }
        // values: this thread reads keys 8t..8t+7 (of each chunk) of value dim 8 nb + g, from the
        // page that holds them. Slots beyond the newest key hold no data yet: keep them out.
        const int in_chunk = 8 * t;
        const int pg = in_chunk >> p.page_shift, off = in_chunk & (p.page_size - 1);
        const size_t voff = (size_t)pg * p.page_size * HD + (size_t)g * p.page_size + off;
        // the running maximum moved for no row of the warp: the accumulators need no rescaling
        const bool same_max = __all_sync(0xffffffffu, alpha[0] == 1.f && alpha[1] == 1.f);
        if (!same_max) {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                o[nb][0] *= alpha[0]; o[nb][1] *= alpha[0];
                o[nb][2] *= alpha[1]; o[nb][3] *= alpha[1];
            }
        }
        if (c0 + NCH * CHUNK - 1 <= hi_tile) {
#pragma unroll
            for (int nb0 = 0; nb0 < NB; nb0 += 4)
#pragma unroll
                for (int ch = 0; ch < NCH; ++ch) {
                    uint4 vf[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        vf[j] = *reinterpret_cast<const uint4*>(vsv[ch] + voff + (size_t)(8 * (nb0 + j)) * p.page_size);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        mma_bf16(o[nb0 + j], pa[ch][0][0], pa[ch][0][1], pa[ch][0][2], pa[ch][0][3], vf[j].x, vf[j].y);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        mma_bf16(o[nb0 + j], pa[ch][1][0], pa[ch][1][1], pa[ch][1][2], pa[ch][1][3], vf[j].z, vf[j].w);
                }
        } else {
            // slots beyond the newest key hold no data yet: keep them out of the product
            unsigned keep[NCH][4];
#pragma unroll
            for (int ch = 0; ch < NCH; ++ch) {
                const int vkey0 = c0 + CHUNK * ch + 8 * t;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const bool lo_ok = vkey0 + 2 * w <= hi_tile, hi_ok = vkey0 + 2 * w + 1 <= hi_tile;
                    keep[ch][w] = (lo_ok ? 0x0000ffffu : 0u) | (hi_ok ? 0xffff0000u : 0u);
                }
            }
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int ch = 0; ch < NCH; ++ch) {
                    uint4 vf = *reinterpret_cast<const uint4*>(vsv[ch] + voff + (size_t)(8 * nb) * p.page_size);
                    vf.x &= keep[ch][0]; vf.y &= keep[ch][1]; vf.z &= keep[ch][2]; vf.w &= keep[ch][3];
                    mma_bf16(o[nb], pa[ch][0][0], pa[ch][0][1], pa[ch][0][2], pa[ch][0][3], vf.x, vf.y);
                    mma_bf16(o[nb], pa[ch][1][0], pa[ch][1][1], pa[ch][1][2], pa[ch][1][3], vf.z, vf.w);
                }
        }
    };
    if (NARROW) {
        // ---- each warp streams chunks c_begin + warp, + 8, ... through a stage of its own: with eight
        // warps a block has eight chunks in flight, and a warp fetches its next chunk when it is done with
        // the one before (more warps hide the copies' latency better than deeper per-warp pipelines did)
        if (my_count > 0 && !first_is_old)
            issue_chunk<HD>(p, my_stages, my_stages + CHUNK * HD, &my_bars[0], my_first * CHUNK, lo_tile,
                            hi_tile, bt, kbase, vbase, page_stride, lane, 32, cached_for(0));
        for (int i = 0; i < my_count; ++i) {
            const int st = i % NARROW_STAGES;
            if (NARROW_STAGES > 1 && i + 1 < my_count) {
                const int nx = (i + 1) % NARROW_STAGES;
                __nv_bfloat16* ks = my_stages + (size_t)nx * STAGE_ELEMS;
                issue_chunk<HD>(p, ks, ks + CHUNK * HD, &my_bars[nx], (my_first + NARROW_WARPS * (i + 1)) * CHUNK,
                                lo_tile, hi_tile, bt, kbase, vbase, page_stride, lane, 32, cached_for(i + 1));
            }
            __syncwarp();
            mbar_wait(&my_bars[st], (unsigned)((i / NARROW_STAGES) & 1), p.status);
            const __nv_bfloat16* ks = my_stages + (size_t)st * STAGE_ELEMS;
            compute(One{}, ks, ks + CHUNK * HD, ks, ks + CHUNK * HD, (my_first + NARROW_WARPS * i) * CHUNK);
            __syncwarp();                         // the stage may be refilled from here on
            if (NARROW_STAGES == 1 && i + 1 < my_count)
                issue_chunk<HD>(p, my_stages, my_stages + CHUNK * HD, &my_bars[0],
                                (my_first + NARROW_WARPS * (i + 1)) * CHUNK, lo_tile, hi_tile, bt, kbase, vbase,
                                page_stride, lane, 32, cached_for(i + 1));
        }
        // ---- combine the warps' partial results through shared memory (stages are free)
        __syncthreads();
        constexpr int RS = HD + 8;                                      // row stride: the warps' stores hit every bank once
        float* red_o = reinterpret_cast<float*>(smem_raw);              // [warp][16][RS]
        float* red_ml = red_o + NARROW_WARPS * 16 * RS;                 // [warp][16][2]
        __shared__ float weight_of[NARROW_WARPS][16], sum_of[16], max_of[16];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = g + 8 * i;
            float* dst = red_o + ((size_t)warp * 16 + r) * RS;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
                *reinterpret_cast<float2*>(dst + 8 * nb + 2 * t) = make_float2(o[nb][2 * i], o[nb][2 * i + 1]);
            if (t == 0) {
                red_ml[((size_t)warp * 16 + r) * 2] = m_run[i];
                red_ml[((size_t)warp * 16 + r) * 2 + 1] = l_run[i];
            }
        }
        __syncthreads();
        // each warp's weight for each row, once (one thread per pair), and each row's maximum and sum
        if (tid < NARROW_WARPS * 16) {
            const int r = tid & 15, w = tid >> 4;
            float m = -INFINITY;
#pragma unroll
            for (int w2 = 0; w2 < NARROW_WARPS; ++w2) m = fmaxf(m, red_ml[((size_t)w2 * 16 + r) * 2]);
            const float mw = red_ml[((size_t)w * 16 + r) * 2];
            weight_of[w][r] = (mw == -INFINITY) ? 0.f : fast_exp2(mw - m);
            if (w == 0) max_of[r] = m;
        }
        __syncthreads();
        if (tid < 16) {
            float l = 0.f;
#pragma unroll
            for (int w = 0; w < NARROW_WARPS; ++w) l += red_ml[((size_t)w * 16 + tid) * 2 + 1] * weight_of[w][tid];
            sum_of[tid] = l;
        }
        if (p.n_splits == 1) __syncthreads();      // the only reader of sum_of among other threads
        const int rows_here = min(16, n_rows - tile_row0);
        const float ln2 = 0.6931471805599453f;
        for (int idx = tid; idx < rows_here * (HD / 4); idx += NARROW_THREADS) {
            const int r = idx / (HD / 4), d = 4 * (idx - r * (HD / 4));
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < NARROW_WARPS; ++w) {
                const float4 v = *reinterpret_cast<const float4*>(red_o + ((size_t)w * 16 + r) * RS + d);
                const float wgt = weight_of[w][r];
                acc.x += v.x * wgt; acc.y += v.y * wgt; acc.z += v.z * wgt; acc.w += v.w * wgt;
            }
            const int row = tile_row0 + r;
            const int tok = row / group, head = kh * group + (row - tok * group);
            if (p.n_splits == 1) {
                const float inv = 1.f / sum_of[r];
                uint2 packed;
                packed.x = pack_bf16(acc.x * inv, acc.y * inv);
                packed.y = pack_bf16(acc.z * inv, acc.w * inv);
                *reinterpret_cast<uint2*>(p.out + (size_t)(q_start + tok) * p.out_stride + (size_t)head * HD + d) = packed;
            } else {
                const size_t base = ((size_t)(q_start + tok) * p.n_heads + head) * p.n_splits + split;
                *reinterpret_cast<float4*>(p.part_o + base * HD + d) = acc;
            }
        }
        if (p.n_splits > 1 && tid < rows_here) {
            const int row = tile_row0 + tid;
            const int tok = row / group, head = kh * group + (row - tok * group);
            const size_t base = ((size_t)(q_start + tok) * p.n_heads + head) * p.n_splits + split;
            p.part_ml[base * 2] = max_of[tid] * ln2;     // the merge kernel works with natural logs
            p.part_ml[base * 2 + 1] = sum_of[tid];
        }
        return;
    }

    // ---- wide tiles: the block streams the chunks two at a time through four shared stages
    auto issue_wide = [&](int ci) {
        if (ci < c_end) {
            __nv_bfloat16* ks = stages + (size_t)((ci - c_begin) % WIDE_STAGES) * STAGE_ELEMS;
            issue_chunk<HD>(p, ks, ks + CHUNK * HD, &bars[(ci - c_begin) % WIDE_STAGES], ci * CHUNK, lo_tile,
                            hi_tile, bt, kbase, vbase, page_stride, tid, MMA_THREADS);
        }
    };
    issue_wide(c_begin);
    issue_wide(c_begin + 1);
    for (int ci = c_begin; ci < c_end; ci += 2) {
        const int i = ci - c_begin;
        __syncthreads();                         // every warp is done with the pair before: its stages are free
        issue_wide(ci + 2);
        issue_wide(ci + 3);
        const int c0 = ci * CHUNK;
        const bool two = ci + 1 < c_end;
        const int span = two ? 2 * CHUNK : CHUNK;
        if (!(warp_has_rows && c0 <= hi_warp && c0 + span - 1 >= lo_warp)) continue;
        const int st0 = i % WIDE_STAGES, st1 = (i + 1) % WIDE_STAGES;
        const __nv_bfloat16* ks0 = stages + (size_t)st0 * STAGE_ELEMS;
        const __nv_bfloat16* ks1 = stages + (size_t)st1 * STAGE_ELEMS;
        mbar_wait(&bars[st0], (unsigned)((i / WIDE_STAGES) & 1), p.status);
        if (two) {
            mbar_wait(&bars[st1], (unsigned)(((i + 1) / WIDE_STAGES) & 1), p.status);
            compute(Two{}, ks0, ks0 + CHUNK * HD, ks1, ks1 + CHUNK * HD, c0);
        } else {
            compute(One{}, ks0, ks0 + CHUNK * HD, ks0, ks0 + CHUNK * HD, c0);
        }
    }

    // each warp writes its own rows; this thread holds columns 8 nb + 2t, + 1 of rows g, g + 8
    if (p.n_splits == 1) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!r_valid[i]) continue;
            const float inv = 1.f / l_run[i];
            __nv_bfloat16* orow = p.out + (size_t)(q_start + r_tok[i]) * p.out_stride +
                                  (size_t)(kh * group + r_head[i]) * HD;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
                *reinterpret_cast<unsigned*>(orow + 8 * nb + 2 * t) =
                    pack_bf16(o[nb][2 * i] * inv, o[nb][2 * i + 1] * inv);
        }
    } else {
        const float ln2 = 0.6931471805599453f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!r_valid[i]) continue;
            const size_t base = ((size_t)(q_start + r_tok[i]) * p.n_heads + kh * group + r_head[i]) *
                                    p.n_splits + split;
            float* po = p.part_o + base * HD;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                po[8 * nb + 2 * t] = o[nb][2 * i];
                po[8 * nb + 2 * t + 1] = o[nb][2 * i + 1];
            }
            if (t == 0) {
                p.part_ml[base * 2] = m_run[i] * ln2;
                p.part_ml[base * 2 + 1] = l_run[i];
            }
        }
    }
}

template <int HD, bool NARROW>
int launch_mma(const MmaAttnParams& p, cudaStream_t stream) {
    const size_t stage_bytes = 2 * (size_t)CHUNK * HD * sizeof(__nv_bfloat16);
    size_t smem = stage_bytes * (NARROW ? NARROW_STAGES * NARROW_WARPS : WIDE_STAGES);
    if (NARROW) {
        const size_t reduce = (size_t)NARROW_WARPS * 16 * (HD + 8 + 2) * sizeof(float);
        if (reduce > smem) smem = reduce;
    }
    if (smem + 1024 > 48 * 1024) {   // the kernel also has a little static shared memory
        cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<HD, NARROW>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) MX_REFUSE("attention: cannot reserve %zu bytes of shared memory", smem);
    }
    dim3 grid(p.n_tiles, p.n_kv_heads, p.n_splits);
    mx_launch_chained(attention_mma_kernel<HD, NARROW>, grid, dim3(NARROW ? NARROW_THREADS : MMA_THREADS), smem, stream, p);
    return mx_launch_status();
}

}  // namespace

extern "C" int mx_attention_merge_bf16(const float* part_o, const float* part_ml, void* out,
                                       int out_stride, int n_tokens, int n_heads, int head_dim,
                                       int n_splits, cudaStream_t stream);

// `narrow` != 0: every tile has at most 16 rows (decode tokens); the eight warps of a block
// share them and take the key chunks in turn. Otherwise tiles are 64 rows, 16 per warp.
extern "C" int mx_paged_attention_mma(const void* q, int q_stride, const void* cache,
                                      long long n_pages, int page_size, const int* block_tables,
                                      int bt_stride, const int* cu_q, const int* context_lens,
                                      const int* tiles, int n_tiles, int narrow, int n_tokens,
                                      int n_heads, int n_kv_heads, int head_dim, int window,
                                      float scale, void* out, int out_stride, int n_splits,
                                      float* scratch, int* status, cudaStream_t stream) {
    if (n_tiles <= 0 || n_tokens <= 0) return MX_OK;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        MX_REFUSE("attention: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    if (head_dim != 64 && head_dim != 128)
        MX_REFUSE("tensor-core attention is built for head_dim 64 and 128, not %d", head_dim);
    if (page_size != 8 && page_size != 16 && page_size != 32)
        MX_REFUSE("tensor-core attention takes pages of 8, 16 or 32 slots, not %d", page_size);
    if (q_stride % 8 != 0 || out_stride % 2 != 0)
        MX_REFUSE("tensor-core attention needs 16-byte aligned query rows (stride %d)", q_stride);
    if (n_splits < 1 || n_splits > 65535) MX_REFUSE("attention: n_splits %d", n_splits);
    if (n_kv_heads > 65535) MX_REFUSE("attention: %d kv heads exceed the grid", n_kv_heads);
    if (n_splits > 1 && scratch == nullptr) MX_REFUSE("attention: split path without scratch memory");
    MmaAttnParams p;
    p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache; p.out = (__nv_bfloat16*)out;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (size_t)n_tokens * n_heads * n_splits * head_dim : nullptr;
    p.block_tables = block_tables; p.cu_q = cu_q; p.context_lens = context_lens; p.tiles = tiles;
    p.status = status; p.n_pages = n_pages; p.n_tiles = n_tiles; p.q_stride = q_stride;
    p.out_stride = out_stride; p.bt_stride = bt_stride; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads;
    p.page_size = page_size; p.page_shift = page_size == 8 ? 3 : (page_size == 16 ? 4 : 5);
    p.window = window; p.n_splits = n_splits;
    p.scale_log2 = scale * 1.4426950408889634f;
    int rc;
    if (head_dim == 64) rc = narrow ? launch_mma<64, true>(p, stream) : launch_mma<64, false>(p, stream);
    else rc = narrow ? launch_mma<128, true>(p, stream) : launch_mma<128, false>(p, stream);
    if (rc != MX_OK || n_splits == 1) return rc;
    return mx_attention_merge_bf16(p.part_o, p.part_ml, out, out_stride, n_tokens, n_heads, head_dim,
                                   n_splits, stream);
}
