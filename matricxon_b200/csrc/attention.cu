// Grouped-query attention of a flattened batch of query tokens over a paged cache.
//
// Visibility rule (the reference's windowed decode attention, app/native/src/mx_attention.c:36-39,
// and its masks, app/architectures/qwen_layers.py:12-17, app/architectures/gemma4_layers.py:17-34):
// the query at absolute position p sees key j iff j <= p and (window == 0 or j > p - window).
// Scores are q.k * scale, softmax is max-subtracted, query head h reads KV head h / (heads / kv heads)
// (app/native/src/mx_attention.c:16-68). Scores, softmax and the weighted sum are float whatever T is.
//
// One block handles (query token, KV head, group of up to 16 query heads, key split). Keys are
// walked in chunks of 32 absolute positions (one key per lane); a split owns a contiguous run of
// chunks. With more than one split each block writes an unnormalised partial (max, sum, weighted
// values) and mx_attention_merge combines them in a fixed order.
//
// Cache layout: [page][2 (k, v)][kv head][page_size x head_dim]: keys as [slot][dim], values
// transposed as [dim][slot]; block_tables[seq][logical page] gives the physical page, negative
// when the request holds none there. page_size must be a multiple of 8.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int ATT_THREADS = 128;
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int KEYS = 32;      // keys per chunk
constexpr int GH = 16;        // query heads per block at most
constexpr int HEADS_PER_WARP = GH / ATT_WARPS;

struct AttnParams {
    const void* q;            // [n_tokens][q_stride], head h at h * head_dim
    const void* cache;
    void* out;                // [n_tokens][out_stride]
    float* part_o;            // [n_tokens][n_heads][n_splits][head_dim]
    float* part_ml;           // [n_tokens][n_heads][n_splits][2]
    const int* block_tables;  // [n_seqs][bt_stride]
    const int* tok_seq;       // [n_tokens]
    const int* positions;     // [n_tokens]
    int* status;
    long long n_pages;
    int q_stride, out_stride, bt_stride;
    int n_heads, n_kv_heads, head_dim, page_size, window, n_splits;
    float scale;
};

template <typename T> struct Vec16;  // 16 bytes of T
template <> struct Vec16<float> { static constexpr int E = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int E = 8; };

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& raw, float* f);
template <>
__device__ __forceinline__ void unpack16<float>(const uint4& raw, float* f) {
    f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y);
    f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
}
template <>
__device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& raw, float* f) {
    const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <typename T, int HD_SLOTS>
__global__ void __launch_bounds__(ATT_THREADS)
paged_attention_kernel(const AttnParams p) {
    constexpr int E = Vec16<T>::E;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int hd = p.head_dim;
    const int cpr = hd / E;                                   // 16-byte chunks per row
    const int swz_mask = (cpr % 8 == 0) ? 7 : 0;
    float* q_s = reinterpret_cast<float*>(smem_raw);          // [GH][hd]
    float* p_s = q_s + GH * hd;                               // [GH][KEYS]
    float* alpha_s = p_s + GH * KEYS;                         // [GH]
    float* m_s = alpha_s + GH;                                // [GH]
    float* l_s = m_s + GH;                                    // [GH]
    uint4* k_s = reinterpret_cast<uint4*>(l_s + GH);          // [KEYS][cpr] (swizzled)
    uint4* v_s = k_s + KEYS * cpr;                            // [KEYS][cpr]

    const int t = blockIdx.x;
    const int group = p.n_heads / p.n_kv_heads;
    const int n_hgroups = (group + GH - 1) / GH;
    const int kh = blockIdx.y / n_hgroups, hg = blockIdx.y - kh * n_hgroups;
    const int split = blockIdx.z;
    const int head0 = kh * group + hg * GH;
    const int gc = min(GH, group - hg * GH);                  // heads this block handles
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    const int seq = p.tok_seq[t];
    if (seq < 0) {  // a padding row of a fixed-size batch: defined output, no cache access
        if (split == 0) {
            T* orow = reinterpret_cast<T*>(p.out) + (size_t)t * p.out_stride + (size_t)head0 * hd;
            for (int i = tid; i < gc * hd; i += ATT_THREADS) orow[i] = from_float<T>(0.f);
        }
        if (p.n_splits > 1) {
            for (int h = 0; h < gc; ++h) {
                const size_t base = ((size_t)t * p.n_heads + head0 + h) * p.n_splits + split;
                for (int d = tid; d < hd; d += ATT_THREADS) p.part_o[base * hd + d] = 0.f;
                if (tid == 0) { p.part_ml[base * 2] = 0.f; p.part_ml[base * 2 + 1] = 1.f; }
            }
        }
        return;
    }
    const int pos = p.positions[t];
    const int hi = pos;
    const int lo = (p.window > 0) ? max(0, pos - p.window + 1) : 0;
    const int first_chunk = lo / KEYS, last_chunk = hi / KEYS;
    const int n_chunks = last_chunk - first_chunk + 1;
    const int per_split = (n_chunks + p.n_splits - 1) / p.n_splits;
    const int c_begin = first_chunk + split * per_split;
    const int c_end = min(last_chunk + 1, c_begin + per_split);

    const T* qrow = reinterpret_cast<const T*>(p.q) + (size_t)t * p.q_stride + (size_t)head0 * hd;
    for (int i = tid; i < gc * hd; i += ATT_THREADS) q_s[i] = to_float(qrow[i]);

    float acc[GH][HD_SLOTS];
#pragma unroll
    for (int h = 0; h < GH; ++h)
#pragma unroll
        for (int s = 0; s < HD_SLOTS; ++s) acc[h][s] = 0.f;
    float m_run[HEADS_PER_WARP], l_run[HEADS_PER_WARP];
#pragma unroll
    for (int hs = 0; hs < HEADS_PER_WARP; ++hs) { m_run[hs] = -INFINITY; l_run[hs] = 0.f; }

    const int* bt = p.block_tables + (size_t)seq * p.bt_stride;
    const T* cache = reinterpret_cast<const T*>(p.cache);
    const size_t head_stride = (size_t)p.page_size * hd;

    for (int ci = c_begin; ci < c_end; ++ci) {
        const int c0 = ci * KEYS;
        // ---- stage the chunk's K rows (zero for keys outside [lo, hi])
        for (int item = tid; item < KEYS * cpr; item += ATT_THREADS) {
            const int j = item / cpr, c = item - j * cpr;
            const int kpos = c0 + j;
            uint4 kv = make_uint4(0, 0, 0, 0);
            if (kpos >= lo && kpos <= hi) {
                const int lp = kpos / p.page_size;
                const long long page = (lp < p.bt_stride) ? bt[lp] : -1;
                if (page < 0 || page >= p.n_pages) {
                    if (c == 0) atomicOr(p.status, MX_STATUS_BAD_PAGE);
                } else {
                    const int off = kpos - lp * p.page_size;
                    const T* kptr = cache + ((size_t)page * 2 * p.n_kv_heads + kh) * head_stride +
                                    (size_t)off * hd + (size_t)c * E;
                    kv = *reinterpret_cast<const uint4*>(kptr);
                }
            }
            k_s[j * cpr + (c ^ (j & swz_mask))] = kv;
        }
        // ---- stage V: global holds [dim][slot]; shared memory wants [key][dim]
        {
            constexpr int GROUPS = KEYS / E;                  // runs of E keys, each inside one page
            T* v_t = reinterpret_cast<T*>(v_s);
            for (int item = tid; item < hd * GROUPS; item += ATT_THREADS) {
                const int d = item / GROUPS, jg = item - d * GROUPS;
                const int kpos0 = c0 + jg * E;
                uint4 raw = make_uint4(0, 0, 0, 0);
                if (kpos0 <= hi && kpos0 + E - 1 >= lo) {
                    const int lp = kpos0 / p.page_size;
                    const long long page = (lp < p.bt_stride) ? bt[lp] : -1;
                    if (page >= 0 && page < p.n_pages) {
                        const int off = kpos0 - lp * p.page_size;
                        const T* vptr = cache + ((size_t)page * 2 * p.n_kv_heads + p.n_kv_heads + kh) * head_stride +
                                        (size_t)d * p.page_size + off;
                        raw = *reinterpret_cast<const uint4*>(vptr);
                    }
                }
                const T* elems = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const int kpos = kpos0 + e;
                    v_t[(size_t)(jg * E + e) * hd + d] =
                        (kpos >= lo && kpos <= hi) ? elems[e] : from_float<T>(0.f);
                }
            }
        }
        __syncthreads();

        // ---- scores: lane = key, this warp's heads are warp, warp + 4, ...
        {
            const int kpos = c0 + lane;
            const bool valid = (kpos >= lo && kpos <= hi);
            float s[HEADS_PER_WARP];
#pragma unroll
            for (int hs = 0; hs < HEADS_PER_WARP; ++hs) s[hs] = 0.f;
            for (int c = 0; c < cpr; ++c) {
                float kf[E];
                unpack16<T>(k_s[lane * cpr + (c ^ (lane & swz_mask))], kf);
#pragma unroll
                for (int hs = 0; hs < HEADS_PER_WARP; ++hs) {
                    const int h = warp + hs * ATT_WARPS;
                    if (h < gc) {
                        const float4* qv = reinterpret_cast<const float4*>(q_s + h * hd + c * E);
#pragma unroll
                        for (int e4 = 0; e4 < E / 4; ++e4) {
                            const float4 qq = qv[e4];
                            s[hs] = fmaf(qq.x, kf[4 * e4 + 0], s[hs]);
                            s[hs] = fmaf(qq.y, kf[4 * e4 + 1], s[hs]);
                            s[hs] = fmaf(qq.z, kf[4 * e4 + 2], s[hs]);
                            s[hs] = fmaf(qq.w, kf[4 * e4 + 3], s[hs]);
                        }
                    }
                }
            }
#pragma unroll
            for (int hs = 0; hs < HEADS_PER_WARP; ++hs) {
                const int h = warp + hs * ATT_WARPS;
                if (h < gc) {
                    const float sv = valid ? s[hs] * p.scale : -INFINITY;
                    const float m_new = fmaxf(m_run[hs], warp_max(sv));
                    const float pj = valid ? expf(sv - m_new) : 0.f;
                    const float alpha = (m_run[hs] == -INFINITY) ? 0.f : expf(m_run[hs] - m_new);
                    l_run[hs] = l_run[hs] * alpha + warp_sum(pj);
                    m_run[hs] = m_new;
                    p_s[h * KEYS + lane] = pj;
                    if (lane == 0) alpha_s[h] = alpha;
                }
            }
        }
        __syncthreads();

        // ---- weighted values: thread = output dim(s), all heads
#pragma unroll
        for (int slot = 0; slot < HD_SLOTS; ++slot) {
            const int d = tid + slot * ATT_THREADS;
            if (d < hd) {
#pragma unroll
                for (int h = 0; h < GH; ++h)
                    if (h < gc) acc[h][slot] *= alpha_s[h];
                const T* vcol = reinterpret_cast<const T*>(v_s) + d;
                for (int j = 0; j < KEYS; j += 4) {
                    const float v0 = to_float(vcol[(size_t)(j + 0) * hd]);
                    const float v1 = to_float(vcol[(size_t)(j + 1) * hd]);
                    const float v2 = to_float(vcol[(size_t)(j + 2) * hd]);
                    const float v3 = to_float(vcol[(size_t)(j + 3) * hd]);
#pragma unroll
                    for (int h = 0; h < GH; ++h) {
                        if (h < gc) {
                            const float4 pp = *reinterpret_cast<const float4*>(p_s + h * KEYS + j);
                            float a = acc[h][slot];
                            a = fmaf(pp.x, v0, a);
                            a = fmaf(pp.y, v1, a);
                            a = fmaf(pp.z, v2, a);
                            a = fmaf(pp.w, v3, a);
                            acc[h][slot] = a;
                        }
                    }
                }
            }
        }
        __syncthreads();
    }

    // ---- hand the running max / sum of each head to every thread
#pragma unroll
    for (int hs = 0; hs < HEADS_PER_WARP; ++hs) {
        const int h = warp + hs * ATT_WARPS;
        if (h < gc && lane == 0) { m_s[h] = m_run[hs]; l_s[h] = l_run[hs]; }
    }
    __syncthreads();

    if (p.n_splits == 1) {
        T* orow = reinterpret_cast<T*>(p.out) + (size_t)t * p.out_stride + (size_t)head0 * hd;
#pragma unroll
        for (int slot = 0; slot < HD_SLOTS; ++slot) {
            const int d = tid + slot * ATT_THREADS;
            if (d < hd) {
#pragma unroll
                for (int h = 0; h < GH; ++h)
                    if (h < gc) orow[(size_t)h * hd + d] = from_float<T>(acc[h][slot] / l_s[h]);
            }
        }
    } else {
#pragma unroll
        for (int h = 0; h < GH; ++h) {
            if (h < gc) {
                const size_t base = ((size_t)t * p.n_heads + head0 + h) * p.n_splits + split;
#pragma unroll
                for (int slot = 0; slot < HD_SLOTS; ++slot) {
                    const int d = tid + slot * ATT_THREADS;
                    if (d < hd) p.part_o[base * hd + d] = acc[h][slot];
                }
                if (tid == 0) { p.part_ml[base * 2] = m_s[h]; p.part_ml[base * 2 + 1] = l_s[h]; }
            }
        }
    }
}

template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part_o,
                                       const float* __restrict__ part_ml, T* __restrict__ out,
                                       int out_stride, int n_heads, int head_dim, int n_splits) {
    // One trip to memory: the maxima and sums of the splits (one per thread, into shared memory) and this
    // thread's value of the first MERGE_AHEAD splits set out together; only then is anything combined.
    // Each split's weight exp(max_s - max) is computed once, by the thread that fetched its maximum.
    // Splits beyond what the shared arrays hold are read where they lie.
    constexpr int MERGE_AHEAD = 16, MERGE_KEPT = 128;
    __shared__ float split_max[MERGE_KEPT], split_sum[MERGE_KEPT], split_weight[MERGE_KEPT];
    __shared__ float total_max, total_sum;
    pdl_trigger();
    pdl_wait();
    part_o = after_wait(part_o);
    part_ml = after_wait(part_ml);
    const int t = blockIdx.x, h = blockIdx.y;
    const size_t base = ((size_t)t * n_heads + h) * n_splits;
    for (int s = threadIdx.x; s < min(n_splits, MERGE_KEPT); s += blockDim.x) {
        split_max[s] = part_ml[(base + s) * 2];
        split_sum[s] = part_ml[(base + s) * 2 + 1];
    }
    const bool mine0 = (int)threadIdx.x < head_dim;
    float ahead[MERGE_AHEAD];
#pragma unroll
    for (int s = 0; s < MERGE_AHEAD; ++s)
        ahead[s] = (s < n_splits && mine0) ? part_o[(base + s) * head_dim + threadIdx.x] : 0.f;
    __syncthreads();
    if (threadIdx.x < 32) {
        // one warp: the maximum over all splits, then every kept split's weight and the weighted sum
        const int lane = threadIdx.x;
        float m = -INFINITY;
        for (int s = lane; s < n_splits; s += 32) m = fmaxf(m, s < MERGE_KEPT ? split_max[s] : part_ml[(base + s) * 2]);
        m = warp_max(m);
        float total = 0.f;
        for (int s = lane; s < n_splits; s += 32) {
            const float ms = s < MERGE_KEPT ? split_max[s] : part_ml[(base + s) * 2];
            const float w = ms == -INFINITY ? 0.f : expf(ms - m);
            if (s < MERGE_KEPT) split_weight[s] = w;
            total += (s < MERGE_KEPT ? split_sum[s] : part_ml[(base + s) * 2 + 1]) * w;
        }
        total = warp_sum(total);
        if (lane == 0) { total_max = m; total_sum = total; }
    }
    __syncthreads();
    const float m = total_max, inv = 1.f / total_sum;
    auto weight_of = [&](int s) {
        if (s < MERGE_KEPT) return split_weight[s];
        const float ms = part_ml[(base + s) * 2];
        return ms == -INFINITY ? 0.f : expf(ms - m);
    };
    for (int d0 = 0; d0 < head_dim; d0 += blockDim.x) {
        const int d = d0 + threadIdx.x;
        const bool mine = d < head_dim;
        float o = 0.f;
        if (d0 == 0) {
#pragma unroll
            // a split without keys has weight 0 and values nobody wrote: it is skipped, not multiplied
            for (int s = 0; s < MERGE_AHEAD; ++s)
                if (s < n_splits && split_weight[s] != 0.f) o += ahead[s] * split_weight[s];
            for (int s = MERGE_AHEAD; s < n_splits; ++s) {
                const float w = weight_of(s);
                if (mine && w != 0.f) o += part_o[(base + s) * head_dim + d] * w;
            }
        } else {
            for (int s = 0; s < n_splits; ++s) {
                const float w = weight_of(s);
                if (mine && w != 0.f) o += part_o[(base + s) * head_dim + d] * w;
            }
        }
        if (mine) out[(size_t)t * out_stride + (size_t)h * head_dim + d] = from_float<T>(o * inv);
    }
}

// The merge for steps with many rows (prompt portions whose keys were shared out): a warp per (token, head),
// eight a block, each lane four neighbouring dims; no shared memory and no barrier. The kernel above, a block
// per pair, is built for the few rows of a decode step and spends 15 us on 6,144 pairs where this one reads
// its 8 MB at the memory's rate. At most MERGE_ROW_SPLITS splits; head_dim a multiple of 4.
constexpr int MERGE_ROW_SPLITS = 8, MERGE_ROW_WARPS = 8;
template <typename T>
__global__ void __launch_bounds__(MERGE_ROW_WARPS * 32)
attention_merge_rows_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, T* __restrict__ out,
                            int out_stride, int n_heads, int head_dim, int n_splits, int n_pairs) {
    pdl_trigger();
    pdl_wait();
    part_o = after_wait(part_o);
    part_ml = after_wait(part_ml);
    const int pair = blockIdx.x * MERGE_ROW_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_pairs) return;
    const int t = pair / n_heads, h = pair - t * n_heads;
    const size_t base = (size_t)pair * n_splits;
    float weight[MERGE_ROW_SPLITS], sums[MERGE_ROW_SPLITS];
    float m = -INFINITY;
#pragma unroll
    for (int s = 0; s < MERGE_ROW_SPLITS; ++s) {
        const float2 ml = s < n_splits ? *reinterpret_cast<const float2*>(part_ml + (base + s) * 2)
                                       : make_float2(-INFINITY, 0.f);
        weight[s] = ml.x;
        sums[s] = ml.y;
        m = fmaxf(m, ml.x);
    }
    float total = 0.f;
#pragma unroll
    for (int s = 0; s < MERGE_ROW_SPLITS; ++s) {
        weight[s] = weight[s] == -INFINITY ? 0.f : expf(weight[s] - m);
        total += sums[s] * weight[s];
    }
    const float inv = 1.f / total;
    for (int d = 4 * lane; d < head_dim; d += 128) {
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < MERGE_ROW_SPLITS; ++s) {
            // a split without keys has weight 0 and values nobody wrote: it is skipped, not multiplied
            if (s < n_splits && weight[s] != 0.f) {
                const float4 v = *reinterpret_cast<const float4*>(part_o + (base + s) * head_dim + d);
                o.x += v.x * weight[s]; o.y += v.y * weight[s]; o.z += v.z * weight[s]; o.w += v.w * weight[s];
            }
        }
        T* dst = out + (size_t)t * out_stride + (size_t)h * head_dim + d;
        dst[0] = from_float<T>(o.x * inv);
        dst[1] = from_float<T>(o.y * inv);
        dst[2] = from_float<T>(o.z * inv);
        dst[3] = from_float<T>(o.w * inv);
    }
}

// Which of the two merges a step takes: the many-row one from 1,024 (token, head) pairs on, where it fits.
template <typename T>
int launch_merge(const float* part_o, const float* part_ml, T* out, int out_stride, int n_tokens, int n_heads,
                 int head_dim, int n_splits, cudaStream_t stream) {
    const long long pairs = (long long)n_tokens * n_heads;
    if (pairs >= 1024 && pairs < (1LL << 31) && n_splits <= MERGE_ROW_SPLITS && head_dim % 4 == 0 &&
        reinterpret_cast<uintptr_t>(part_o) % 16 == 0) {
        const int blocks = (int)((pairs + MERGE_ROW_WARPS - 1) / MERGE_ROW_WARPS);
        mx_launch_chained(attention_merge_rows_kernel<T>, dim3(blocks), dim3(MERGE_ROW_WARPS * 32), 0, stream, part_o,
                          part_ml, out, out_stride, n_heads, head_dim, n_splits, (int)pairs);
        return mx_launch_status();
    }
    mx_launch_chained(attention_merge_kernel<T>, dim3(n_tokens, n_heads), dim3(128), 0, stream, part_o, part_ml, out,
                      out_stride, n_heads, head_dim, n_splits);
    return mx_launch_status();
}

template <typename T>
size_t attention_smem_bytes(int head_dim) {
    return (size_t)GH * head_dim * 4 + (size_t)GH * KEYS * 4 + 3 * GH * 4 +
           2 * (size_t)KEYS * head_dim * sizeof(T);
}

template <typename T, int HD_SLOTS>
int launch_attention(const AttnParams& p, int n_tokens, cudaStream_t stream) {
    const size_t smem = attention_smem_bytes<T>(p.head_dim);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(paged_attention_kernel<T, HD_SLOTS>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) MX_REFUSE("attention: cannot reserve %zu bytes of shared memory", smem);
    }
    const int group = p.n_heads / p.n_kv_heads;
    const int n_hgroups = (group + GH - 1) / GH;
    dim3 grid(n_tokens, p.n_kv_heads * n_hgroups, p.n_splits);
    paged_attention_kernel<T, HD_SLOTS><<<grid, ATT_THREADS, smem, stream>>>(p);
    int rc = mx_launch_status();
    if (rc != MX_OK || p.n_splits == 1) return rc;
    return launch_merge<T>(p.part_o, p.part_ml, (T*)p.out, p.out_stride, n_tokens, p.n_heads, p.head_dim, p.n_splits,
                           stream);
}

}  // namespace

// Bytes of scratch the split path needs: partial values plus (max, sum) per split.
extern "C" long long mx_attention_scratch_bytes(int n_tokens, int n_heads, int head_dim, int n_splits) {
    if (n_splits <= 1) return 0;
    return (long long)n_tokens * n_heads * n_splits * (head_dim + 2) * (long long)sizeof(float);
}

extern "C" int mx_paged_attention(const void* q, int dtype, int q_stride, const void* cache,
                                  long long n_pages, int page_size, const int* block_tables,
                                  int bt_stride, const int* tok_seq, const int* positions,
                                  int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                  int window, float scale, void* out, int out_stride,
                                  int n_splits, float* scratch, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        MX_REFUSE("attention: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    if (head_dim % 16 != 0 || head_dim < 16 || head_dim > 256)
        MX_REFUSE("attention: head_dim %d is not a multiple of 16 in [16, 256]", head_dim);
    if (page_size <= 0 || page_size % 8 != 0)
        MX_REFUSE("attention: page size %d is not a positive multiple of 8", page_size);
    if (n_splits < 1) MX_REFUSE("attention: n_splits %d", n_splits);
    if (n_splits > 1 && scratch == nullptr) MX_REFUSE("attention: split path without scratch memory");
    if (n_splits > 65535) MX_REFUSE("attention: %d splits exceed the grid's third dimension", n_splits);
    AttnParams p;
    p.q = q; p.cache = cache; p.out = out;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (size_t)n_tokens * n_heads * n_splits * head_dim : nullptr;
    p.block_tables = block_tables; p.tok_seq = tok_seq; p.positions = positions; p.status = status;
    p.n_pages = n_pages; p.q_stride = q_stride; p.out_stride = out_stride; p.bt_stride = bt_stride;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.page_size = page_size;
    p.window = window; p.n_splits = n_splits; p.scale = scale;
    const bool two = head_dim > ATT_THREADS;
    if (dtype == MX_DTYPE_F32)
        return two ? launch_attention<float, 2>(p, n_tokens, stream) : launch_attention<float, 1>(p, n_tokens, stream);
    return two ? launch_attention<__nv_bfloat16, 2>(p, n_tokens, stream)
               : launch_attention<__nv_bfloat16, 1>(p, n_tokens, stream);
}

// The merge step alone, for kernels in other files that write partials in this layout.
extern "C" int mx_attention_merge_bf16(const float* part_o, const float* part_ml, void* out,
                                       int out_stride, int n_tokens, int n_heads, int head_dim,
                                       int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    return launch_merge<__nv_bfloat16>(part_o, part_ml, (__nv_bfloat16*)out, out_stride, n_tokens, n_heads, head_dim,
                                       n_splits, stream);
}

// ---------------------------------------------------------------------------------------------
// The same attention for callers that cannot allocate: scratch lives in the library image.
// See no_alloc.h for who needs this and for the rules of use.
#include "no_alloc.h"

namespace {

constexpr int MX_MAX_DEVICES = 64;

// Reserved on every device that loads this library, until the process exits.
static __device__ __align__(256) float g_static_attention_scratch[MX_STATIC_ATTENTION_SCRATCH_BYTES / sizeof(float)];

// In host code the array's name is only a handle for the runtime, not a device pointer; the
// address a kernel can use comes from cudaGetSymbolAddress, once per device.
float* g_static_scratch_address[MX_MAX_DEVICES] = {nullptr};

int static_scratch_for_current_device(float** address) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) {
        mx_set_error("static attention: cudaGetDevice failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    if (device < 0 || device >= MX_MAX_DEVICES)
        MX_REFUSE("static attention: device ordinal %d is beyond the %d this library tracks", device, MX_MAX_DEVICES);
    if (g_static_scratch_address[device] == nullptr) {
        void* found = nullptr;
        e = cudaGetSymbolAddress(&found, g_static_attention_scratch);
        if (e != cudaSuccess || found == nullptr) {
            mx_set_error("static attention: cudaGetSymbolAddress failed on device %d: %s", device,
                         cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : MX_ERR_ARGUMENT;
        }
        g_static_scratch_address[device] = static_cast<float*>(found);
    }
    *address = g_static_scratch_address[device];
    return MX_OK;
}

}  // namespace

extern "C" long long mx_static_attention_scratch_bytes(void) { return MX_STATIC_ATTENTION_SCRATCH_BYTES; }

extern "C" int mx_paged_attention_static(const void* q, int dtype, int q_stride, const void* cache,
                                         long long n_pages, int page_size, const int* block_tables,
                                         int bt_stride, const int* tok_seq, const int* positions,
                                         int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                         int window, float scale, void* out, int out_stride,
                                         int n_splits, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    // sizes are checked before they are multiplied: a non-positive one would make `need` negative
    // and slip under the limit
    if (n_splits < 1 || n_splits > 65535) MX_REFUSE("static attention: n_splits %d is not in 1..65535", n_splits);
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        MX_REFUSE("static attention: %d heads over %d kv heads", n_heads, n_kv_heads);
    if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 256)
        MX_REFUSE("static attention: head_dim %d is not a multiple of 16 up to 256", head_dim);
    const long long need = mx_attention_scratch_bytes(n_tokens, n_heads, head_dim, n_splits);
    if (need < 0 || need > MX_STATIC_ATTENTION_SCRATCH_BYTES)
        MX_REFUSE("static attention: %d tokens x %d heads x %d splits x head_dim %d need %lld bytes "
                  "of scratch, the built-in array holds %lld; use fewer splits or tokens per call",
                  n_tokens, n_heads, n_splits, head_dim, need, (long long)MX_STATIC_ATTENTION_SCRATCH_BYTES);
    float* scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != MX_OK) return rc;
    return mx_paged_attention(q, dtype, q_stride, cache, n_pages, page_size, block_tables, bt_stride,
                              tok_seq, positions, n_tokens, n_heads, n_kv_heads, head_dim, window,
                              scale, out, out_stride, n_splits, scratch, status, stream);
}
