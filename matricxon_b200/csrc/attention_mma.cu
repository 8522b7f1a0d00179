// Tensor-core paged attention for bfloat16: prefill portions and decode tokens in one kernel.
//
// Same mathematics and visibility rule as attention.cu (query at p sees key j iff j <= p and
// (window == 0 or j > p - window); scores q.k * scale; float softmax; query head h reads KV
// head h / group), cf. app/native/src/mx_attention.c:16-68 and
// app/architectures/qwen_layers.py:12-17,94-100.
//
// Rows. For one sequence and one KV head, the query rows are the pairs (token, head in
// group), token-major: row r = t * group + h. A warp owns 16 consecutive rows (an MMA M
// tile); with grouped queries those rows sit on one or two tokens, so they share nearly the
// same causal limit and every key they load is used by all of them. A decode token is the
// case of `group` rows; a prompt portion of q tokens has q * group rows.
//
// Work. One warp = one work item (row tile, KV head, key split); warps never talk to each
// other, there is no shared memory and no block barrier. Keys are walked in chunks of 32
// absolute positions. Everything stays in registers, read from global memory with 16-byte
// loads:
//   * S = Q K^T: mma.sync.m16n8k16 (bf16 in, float out). The contraction runs over head
//     dims in a permuted order chosen so that each thread's A and B fragments are 16
//     contiguous bytes of a Q row and of a K row.
//   * the 8 score columns of an MMA are assigned to keys so that, after the four MMAs of a
//     chunk, thread t of a quad holds the scores of keys 8t..8t+7 of the chunk: exactly the
//     A fragment the P V product needs, with values stored transposed ([dim][slot]) so that
//     its B fragment is again 16 contiguous bytes.
// With more than one split a work item writes unnormalised partials (max, sum, values) in
// the layout of attention.cu, and that file's merge kernel combines them.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int MMA_WARPS = 4;
constexpr int MMA_THREADS = MMA_WARPS * 32;
constexpr int CHUNK = 32;

struct MmaAttnParams {
    const __nv_bfloat16* q;      // [tokens][q_stride], head h at h * HD
    const __nv_bfloat16* cache;  // [page][2][kv head][page_size * HD]: K [slot][dim], V [dim][slot]
    __nv_bfloat16* out;          // [tokens][out_stride]
    float* part_o;               // [tokens][heads][splits][HD]
    float* part_ml;              // [tokens][heads][splits][2]
    const int* block_tables;     // [seqs][bt_stride]
    const int* cu_q;             // [seqs + 1] first token row of each sequence
    const int* context_lens;     // [seqs] tokens cached before this step
    const int* tiles;            // [n_tiles][2]: (sequence, first row of the 16-row tile)
    int* status;
    long long n_pages;
    int n_tiles, q_stride, out_stride, bt_stride;
    int n_heads, n_kv_heads, page_size, window, n_splits;
    float scale_log2;            // scale * log2(e)
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2,
                                         unsigned a3, unsigned b0, unsigned b1) {
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

template <int HD>
__global__ void __launch_bounds__(MMA_THREADS)
attention_mma_kernel(const MmaAttnParams p) {
    constexpr int KB = HD / 32;   // 32-wide blocks of the head dim (two MMA k-steps each)
    constexpr int NB = HD / 8;    // 8-wide output column blocks
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const long long item = (long long)blockIdx.x * MMA_WARPS + (threadIdx.x >> 5);
    const long long n_items = (long long)p.n_tiles * p.n_kv_heads * p.n_splits;
    if (item >= n_items) return;
    const int split = (int)(item % p.n_splits);
    const int kh = (int)((item / p.n_splits) % p.n_kv_heads);
    const int tile = (int)(item / ((long long)p.n_splits * p.n_kv_heads));

    const int seq = p.tiles[2 * tile], row0 = p.tiles[2 * tile + 1];
    const int group = p.n_heads / p.n_kv_heads;
    const int q_start = p.cu_q[seq];
    const int q_len = p.cu_q[seq + 1] - q_start;
    const int ctx = p.context_lens[seq];
    const int n_rows = q_len * group;
    if (row0 >= n_rows) return;
    const int last_row = min(row0 + 15, n_rows - 1);

    // the two rows this thread owns: row0 + g and row0 + g + 8
    int r_tok[2], r_head[2], r_pos[2], r_lo[2];
    bool r_valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = row0 + g + 8 * i;
        r_valid[i] = r < n_rows;
        const int rr = r_valid[i] ? r : last_row;
        r_tok[i] = rr / group;
        r_head[i] = rr - r_tok[i] * group;
        r_pos[i] = ctx + r_tok[i];
        r_lo[i] = p.window > 0 ? max(0, r_pos[i] - p.window + 1) : 0;
    }
    const int first_tok = row0 / group, last_tok = last_row / group;
    const int hi_tile = ctx + last_tok;
    const int lo_tile = p.window > 0 ? max(0, ctx + first_tok - p.window + 1) : 0;
    const int first_chunk = lo_tile / CHUNK, last_chunk = hi_tile / CHUNK;
    const int n_chunks = last_chunk - first_chunk + 1;
    const int per_split = (n_chunks + p.n_splits - 1) / p.n_splits;
    const int c_begin = first_chunk + split * per_split;
    const int c_end = min(last_chunk + 1, c_begin + per_split);

    // Q fragments: 16 bytes of each owned row per 32-wide block
    uint4 qf[2][KB];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const __nv_bfloat16* qrow = p.q + (size_t)(q_start + r_tok[i]) * p.q_stride +
                                    (size_t)(kh * group + r_head[i]) * HD;
#pragma unroll
        for (int b = 0; b < KB; ++b)
            qf[i][b] = r_valid[i] ? *reinterpret_cast<const uint4*>(qrow + 32 * b + 8 * t)
                                  : make_uint4(0, 0, 0, 0);
    }

    float o[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    const int* bt = p.block_tables + (size_t)seq * p.bt_stride;
    const size_t head_stride = (size_t)p.page_size * HD;
    const __nv_bfloat16* kbase = p.cache + (size_t)kh * head_stride;
    const __nv_bfloat16* vbase = p.cache + (size_t)(p.n_kv_heads + kh) * head_stride;
    const size_t page_stride = 2 * (size_t)p.n_kv_heads * head_stride;

    for (int ci = c_begin; ci < c_end; ++ci) {
        const int c0 = ci * CHUNK;
        // ---- scores: block b of the chunk gives this thread keys 8t + 2b, 8t + 2b + 1
        float s[4][4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            s[b][0] = s[b][1] = s[b][2] = s[b][3] = 0.f;
            // column g of block b is key 8 * (g / 2) + 2b + (g % 2): this thread supplies its K row
            const int key = c0 + 8 * (g >> 1) + 2 * b + (g & 1);
            const __nv_bfloat16* krow = nullptr;
            if (key >= lo_tile && key <= hi_tile) {
                const int lp = key / p.page_size;
                const long long page = lp < p.bt_stride ? bt[lp] : -1;
                if (page >= 0 && page < p.n_pages)
                    krow = kbase + (size_t)page * page_stride + (size_t)(key - lp * p.page_size) * HD;
                else if (t == 0)
                    atomicOr(p.status, MX_STATUS_BAD_PAGE);
            }
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint4 kf = krow ? *reinterpret_cast<const uint4*>(krow + 32 * kb + 8 * t)
                                      : make_uint4(0, 0, 0, 0);
                mma_bf16(s[b], qf[0][kb].x, qf[1][kb].x, qf[0][kb].y, qf[1][kb].y, kf.x, kf.y);
                mma_bf16(s[b], qf[0][kb].z, qf[1][kb].z, qf[0][kb].w, qf[1][kb].w, kf.z, kf.w);
            }
        }
        // ---- mask, running max and sum (rows g and g + 8), probabilities in place
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = e >> 1;
                const int key = c0 + 8 * t + 2 * b + (e & 1);
                const bool visible = r_valid[i] && key <= r_pos[i] && key >= r_lo[i];
                s[b][e] = visible ? s[b][e] * p.scale_log2 : -INFINITY;
                m_new[i] = fmaxf(m_new[i], s[b][e]);
            }
        float alpha[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
            m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
            alpha[i] = (m_run[i] == -INFINITY) ? 0.f : exp2f(m_run[i] - m_new[i]);
        }
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = e >> 1;
                const float pv = (s[b][e] == -INFINITY) ? 0.f : exp2f(s[b][e] - m_new[i]);
                s[b][e] = pv;
                sum[i] += pv;
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
            sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
            l_run[i] = l_run[i] * alpha[i] + sum[i];
            m_run[i] = m_new[i];
        }
        // P as A fragments: step st uses blocks 2 st and 2 st + 1
        unsigned pa[2][4];
#pragma unroll
        for (int st = 0; st < 2; ++st) {
            pa[st][0] = pack_bf16(s[2 * st][0], s[2 * st][1]);
            pa[st][1] = pack_bf16(s[2 * st][2], s[2 * st][3]);
            pa[st][2] = pack_bf16(s[2 * st + 1][0], s[2 * st + 1][1]);
            pa[st][3] = pack_bf16(s[2 * st + 1][2], s[2 * st + 1][3]);
        }
        // ---- values: this thread reads keys 8t..8t+7 of value dim 8 nb + g
        const int vkey0 = c0 + 8 * t;
        const __nv_bfloat16* vrow = nullptr;
        if (vkey0 <= hi_tile && vkey0 + 7 >= lo_tile) {
            const int lp = vkey0 / p.page_size;
            const long long page = lp < p.bt_stride ? bt[lp] : -1;
            if (page >= 0 && page < p.n_pages)
                vrow = vbase + (size_t)page * page_stride + (vkey0 - lp * p.page_size);
        }
        // slots beyond the newest key hold no data yet: keep them out of the product
        unsigned keep[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
        if (vkey0 + 7 > hi_tile) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const bool lo_ok = vkey0 + 2 * w <= hi_tile, hi_ok = vkey0 + 2 * w + 1 <= hi_tile;
                keep[w] = (lo_ok ? 0x0000ffffu : 0u) | (hi_ok ? 0xffff0000u : 0u);
            }
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            uint4 vf = make_uint4(0, 0, 0, 0);
            if (vrow) vf = *reinterpret_cast<const uint4*>(vrow + (size_t)(8 * nb + g) * p.page_size);
            vf.x &= keep[0]; vf.y &= keep[1]; vf.z &= keep[2]; vf.w &= keep[3];
            o[nb][0] *= alpha[0]; o[nb][1] *= alpha[0];
            o[nb][2] *= alpha[1]; o[nb][3] *= alpha[1];
            mma_bf16(o[nb], pa[0][0], pa[0][1], pa[0][2], pa[0][3], vf.x, vf.y);
            mma_bf16(o[nb], pa[1][0], pa[1][1], pa[1][2], pa[1][3], vf.z, vf.w);
        }
    }

    // ---- write out: this thread holds columns 8 nb + 2t, + 1 of rows g and g + 8
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
                // the merge kernel works with natural-log maxima
                p.part_ml[base * 2] = m_run[i] * ln2;
                p.part_ml[base * 2 + 1] = l_run[i];
            }
        }
    }
}

}  // namespace

extern "C" int mx_attention_merge_bf16(const float* part_o, const float* part_ml, void* out,
                                       int out_stride, int n_tokens, int n_heads, int head_dim,
                                       int n_splits, cudaStream_t stream);

extern "C" int mx_paged_attention_mma(const void* q, int q_stride, const void* cache,
                                      long long n_pages, int page_size, const int* block_tables,
                                      int bt_stride, const int* cu_q, const int* context_lens,
                                      const int* tiles, int n_tiles, int n_tokens, int n_heads,
                                      int n_kv_heads, int head_dim, int window, float scale,
                                      void* out, int out_stride, int n_splits, float* scratch,
                                      int* status, cudaStream_t stream) {
    if (n_tiles <= 0 || n_tokens <= 0) return MX_OK;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        MX_REFUSE("attention: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    if (head_dim != 64 && head_dim != 128)
        MX_REFUSE("tensor-core attention is built for head_dim 64 and 128, not %d", head_dim);
    if (page_size <= 0 || page_size % 8 != 0)
        MX_REFUSE("attention: page size %d is not a positive multiple of 8", page_size);
    if (q_stride % 8 != 0 || out_stride % 2 != 0)
        MX_REFUSE("tensor-core attention needs 16-byte aligned query rows (stride %d)", q_stride);
    if (n_splits < 1 || n_splits > 65535) MX_REFUSE("attention: n_splits %d", n_splits);
    if (n_splits > 1 && scratch == nullptr) MX_REFUSE("attention: split path without scratch memory");
    MmaAttnParams p;
    p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache; p.out = (__nv_bfloat16*)out;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (size_t)n_tokens * n_heads * n_splits * head_dim : nullptr;
    p.block_tables = block_tables; p.cu_q = cu_q; p.context_lens = context_lens; p.tiles = tiles;
    p.status = status; p.n_pages = n_pages; p.n_tiles = n_tiles; p.q_stride = q_stride;
    p.out_stride = out_stride; p.bt_stride = bt_stride; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads;
    p.page_size = page_size; p.window = window; p.n_splits = n_splits;
    p.scale_log2 = scale * 1.4426950408889634f;
    const long long n_items = (long long)n_tiles * n_kv_heads * n_splits;
    const long long blocks = (n_items + MMA_WARPS - 1) / MMA_WARPS;
    if (blocks > 2147483647LL) MX_REFUSE("attention: too many work items");
    if (head_dim == 64)
        attention_mma_kernel<64><<<(unsigned)blocks, MMA_THREADS, 0, stream>>>(p);
    else
        attention_mma_kernel<128><<<(unsigned)blocks, MMA_THREADS, 0, stream>>>(p);
    int rc = mx_launch_status();
    if (rc != MX_OK || n_splits == 1) return rc;
    return mx_attention_merge_bf16(p.part_o, p.part_ml, out, out_stride, n_tokens, n_heads, head_dim,
                                   n_splits, stream);
}
