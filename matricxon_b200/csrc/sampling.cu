// Next-token choice on the GPU, one block per row of float32 logits.
//
// Pipeline of the reference's sampler (app/runtime/sampler.py:93-129; one-pass C version
// app/native/src/mx_sample.c:51-108): repeat penalty on already generated ids (positive
// scores divided, negative multiplied); temperature <= 0 means argmax and nothing else runs;
// otherwise scores / temperature, top-k keeps every score >= the k-th largest (ties kept),
// softmax weights exp(x - max) over what is kept, top-p keeps a candidate iff the weight of
// the candidates ranked before it is <= p * total (always the best one), and the draw is the
// inverse CDF in vocabulary order: the first index whose running weight exceeds u * total.
//
// Weights are turned into 36-bit fixed point so every sum is an integer sum: the result does
// not depend on the order of additions, hence not on the launch shape or the batch. The k-th
// largest score and the top-p cut are found by radix selection over the order-preserving
// integer image of the floats (four 8-bit passes), by count and by weight.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int SAMPLE_THREADS = 1024;
constexpr double FIXED_ONE = 68719476736.0;  // 2^36

__device__ __forceinline__ unsigned order_key(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long fixed_weight(float x, float peak) {
    return (unsigned long long)((double)expf(x - peak) * FIXED_ONE);
}

struct ArgMax {
    float value;
    int index;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
    return a;
}

__device__ ArgMax block_argmax(ArgMax v, ArgMax* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax other;
        other.value = __shfl_xor_sync(0xffffffffu, v.value, o);
        other.index = __shfl_xor_sync(0xffffffffu, v.index, o);
        v = better(v, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    ArgMax best = scratch[0];
    for (int w = 1; w < SAMPLE_THREADS / 32; ++w) best = better(best, scratch[w]);
    return best;
}

__device__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    unsigned long long total = 0;
    for (int w = 0; w < SAMPLE_THREADS / 32; ++w) total += scratch[w];
    return total;
}

// Radix selection from the top. With BY_WEIGHT the histogram holds fixed-point weights and
// `rank` is a weight; otherwise it holds counts. Returns the key of the element at which the
// descending cumulative (count or weight) first reaches `rank`; 0 if the total is below it.
template <bool BY_WEIGHT>
__device__ unsigned radix_select(const float* work, int vocab, unsigned floor_key, float peak,
                                 unsigned long long rank, unsigned long long* hist,
                                 unsigned* shared_u32, unsigned long long* shared_u64) {
    unsigned prefix = 0, mask = 0;
    for (int pass = 3; pass >= 0; --pass) {
        for (int b = threadIdx.x; b < 256; b += SAMPLE_THREADS) hist[b] = 0;
        __syncthreads();
        // Scores of one row sit in a narrow range, so most of them share a bucket in the upper passes:
        // the lanes of a warp that meet in a bucket add up among themselves first (integer sums: the order
        // does not matter) and one of them does the atomic.
        const int lane = threadIdx.x & 31;
        for (int i0 = 0; i0 < vocab; i0 += SAMPLE_THREADS) {        // the same trip count for every lane
            const int i = i0 + threadIdx.x;
            const float x = i < vocab ? work[i] : 0.f;
            const unsigned key = order_key(x);
            const bool counted = i < vocab && key >= floor_key && (key & mask) == prefix;
            const unsigned bucket = counted ? ((key >> (8 * pass)) & 255u) : 0xffffffffu;
            const unsigned peers = __match_any_sync(0xffffffffu, bucket);
            unsigned long long add = 1ull;
            if (BY_WEIGHT) {
                const unsigned long long w = counted ? fixed_weight(x, peak) : 0ull;
                const unsigned lo = __reduce_add_sync(peers, (unsigned)(w & 0xffffu));
                const unsigned mid = __reduce_add_sync(peers, (unsigned)((w >> 16) & 0xffffu));
                const unsigned hi = __reduce_add_sync(peers, (unsigned)(w >> 32));
                add = (unsigned long long)lo + ((unsigned long long)mid << 16) + ((unsigned long long)hi << 32);
            } else {
                add = (unsigned long long)__popc(peers);
            }
            if (counted && lane == __ffs(peers) - 1) atomicAdd(&hist[bucket], add);
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // warp 0 walks the histogram from the top: lane l owns buckets 255 - 8 l ... 248 - 8 l
            const int top = 255 - 8 * lane;
            unsigned long long mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) mine += hist[top - j];
            unsigned long long incl = mine;                  // sum over this lane and the lanes above it in rank
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            const bool here = incl >= rank && incl - mine < rank;   // the rank falls among this lane's buckets
            if (here) {
                unsigned long long before = incl - mine;
                int chosen = top;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    chosen = top - j;
                    if (before + hist[chosen] >= rank) break;
                    before += hist[chosen];
                }
                shared_u32[0] = (unsigned)(chosen + 1);
                shared_u64[0] = rank - before;
            }
            const unsigned long long total = __shfl_sync(0xffffffffu, incl, 31);
            if (lane == 0 && total < rank) shared_u32[0] = 0u;   // 0 means: total below rank
        }
        __syncthreads();
        if (shared_u32[0] == 0) return 0u;
        prefix |= (shared_u32[0] - 1u) << (8 * pass);
        mask |= 0xffu << (8 * pass);
        rank = shared_u64[0];
        __syncthreads();
    }
    return prefix;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ repeat_penalty,
              const float* __restrict__ uniform, const int* __restrict__ penalty_offsets,
              const int* __restrict__ penalty_ids, const int* __restrict__ pending_ids,
              float* __restrict__ work_all, int* __restrict__ out_tokens, int mark_words) {
    __shared__ ArgMax arg_scratch[SAMPLE_THREADS / 32];
    __shared__ unsigned long long sum_scratch[SAMPLE_THREADS / 32];
    __shared__ unsigned long long hist[256];
    __shared__ unsigned shared_u32[2];
    __shared__ unsigned long long shared_u64[2];
    __shared__ int found_index;

    const int row = blockIdx.x;
    const float* src = logits + (size_t)row * row_stride;
    float* work = work_all + (size_t)row * vocab;
    const int tid = threadIdx.x;

    if (temperature[row] <= 0.f && mark_words > 0) {
        // Greedy: one pass over the logits where they lie. The penalised ids are marked in a bitmap in
        // shared memory and left out of the pass; their adjusted scores are candidates of their own (each
        // from the raw score, so an id that is both listed and pending is penalised once).
        extern __shared__ unsigned marked[];
        const float penalty = repeat_penalty[row];
        const int first = penalty_offsets[row], last = penalty_offsets[row + 1];
        const int pending = pending_ids != nullptr ? pending_ids[row] : -1;
        const bool penalised = penalty != 1.0f && (last > first || pending >= 0);
        ArgMax best = {-INFINITY, 0x7fffffff};
        if (penalised) {
            for (int w = tid; w < mark_words; w += SAMPLE_THREADS) marked[w] = 0u;
            __syncthreads();
            for (int j = first + tid; j <= last; j += SAMPLE_THREADS) {
                const int id = j < last ? penalty_ids[j] : pending;
                if (id >= 0 && id < vocab) {
                    atomicOr(&marked[id >> 5], 1u << (id & 31));
                    const float x = src[id];
                    best = better(best, ArgMax{x > 0.f ? x / penalty : x * penalty, id});
                }
            }
            __syncthreads();
            // every score is loaded whatever the bitmap says (loads that wait for a test cannot overlap)
#pragma unroll 8
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
                const float x = src[i];
                const bool out_of_it = (marked[i >> 5] >> (i & 31)) & 1u;
                best = better(best, ArgMax{out_of_it ? -INFINITY : x, i});
            }
        } else {
#pragma unroll 8
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) best = better(best, ArgMax{src[i], i});
        }
        best = block_argmax(best, arg_scratch);
        if (tid == 0) out_tokens[row] = best.index;
        return;
    }

    for (int i = tid; i < vocab; i += SAMPLE_THREADS) work[i] = src[i];
    __syncthreads();
    const float penalty = repeat_penalty[row];
    if (penalty != 1.0f) {
        for (int j = penalty_offsets[row] + tid; j < penalty_offsets[row + 1]; j += SAMPLE_THREADS) {
            const int id = penalty_ids[j];                   // ids are distinct within a row
            if (id >= 0 && id < vocab) {
                const float x = work[id];
                work[id] = x > 0.f ? x / penalty : x * penalty;
            }
        }
        if (pending_ids != nullptr) {
            // One more generated id that the host does not know yet (the token the step before this one
            // chose, still on the device): penalised like the others unless it is one of them already.
            const int id = pending_ids[row];
            int listed = 0;
            for (int j = penalty_offsets[row] + tid; j < penalty_offsets[row + 1]; j += SAMPLE_THREADS)
                listed |= penalty_ids[j] == id;
            listed = __syncthreads_or(listed);      // also orders the penalties above before the one below
            if (!listed && tid == 0 && id >= 0 && id < vocab) {
                const float x = work[id];
                work[id] = x > 0.f ? x / penalty : x * penalty;
            }
        }
        __syncthreads();
    }

    const float temp = temperature[row];
    if (temp <= 0.f) {
        ArgMax best = {-INFINITY, 0x7fffffff};
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) best = better(best, ArgMax{work[i], i});
        best = block_argmax(best, arg_scratch);
        if (tid == 0) out_tokens[row] = best.index;
        return;
    }

    ArgMax best = {-INFINITY, 0x7fffffff};
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float x = work[i] / temp;
        work[i] = x;
        best = better(best, ArgMax{x, i});
    }
    best = block_argmax(best, arg_scratch);
    const float peak = best.value;

    unsigned floor_key = 0;
    const int k = top_k[row];
    if (k > 0 && k < vocab)
        floor_key = radix_select<false>(work, vocab, 0u, peak, (unsigned long long)k, hist, shared_u32, shared_u64);

    const float p = top_p[row];
    if (p < 1.0f) {
        unsigned long long local = 0;
        for (int i = tid; i < vocab; i += SAMPLE_THREADS)
            if (order_key(work[i]) >= floor_key) local += fixed_weight(work[i], peak);
        const unsigned long long total = block_sum_u64(local, sum_scratch);
        const unsigned long long limit = (unsigned long long)((double)p * (double)total);
        const unsigned cut = radix_select<true>(work, vocab, floor_key, peak, limit + 1ull, hist, shared_u32, shared_u64);
        if (cut > floor_key) floor_key = cut;
    }

    // inverse CDF in vocabulary order over what is kept: warp w owns the contiguous segment
    // [w * seg, (w + 1) * seg) and reads it 32 neighbours at a time
    const int lane = tid & 31, warp = tid >> 5;
    const int seg = ((vocab + SAMPLE_THREADS / 32 - 1) / (SAMPLE_THREADS / 32) + 31) & ~31;
    const int begin = min(vocab, warp * seg), end = min(vocab, begin + seg);
    unsigned long long local = 0;
    for (int i = begin + lane; i < end; i += 32)
        if (order_key(work[i]) >= floor_key) local += fixed_weight(work[i], peak);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    __syncthreads();
    if (lane == 0) sum_scratch[warp] = local;
    if (tid == 0) found_index = 0x7fffffff;
    __syncthreads();
    unsigned long long running = 0, total = 0;
    for (int w = 0; w < SAMPLE_THREADS / 32; ++w) {
        if (w < warp) running += sum_scratch[w];
        total += sum_scratch[w];
    }
    const double target = (double)uniform[row] * (double)total;
    int last_kept = -1;
    bool found = false;
    for (int i0 = begin; i0 < end && !found; i0 += 32) {              // a warp-uniform loop
        const int i = i0 + lane;
        const bool kept = i < end && order_key(work[i]) >= floor_key;
        const unsigned any = __ballot_sync(0xffffffffu, kept);
        if (any == 0u) continue;
        last_kept = max(last_kept, i0 + 31 - __clz(any));
        unsigned long long incl = kept ? fixed_weight(work[i], peak) : 0ull;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, kept && (double)(running + incl) > target);
        if (hit != 0u) {
            if (lane == 0) atomicMin(&found_index, i0 + __ffs(hit) - 1);
            found = true;
        }
        running += __shfl_sync(0xffffffffu, incl, 31);
    }
    __syncthreads();
    if (found_index == 0x7fffffff) {
        // u * total rounded up to the total: the reference falls back to the last candidate
        ArgMax last = {(float)last_kept, -last_kept};
        last = block_argmax(last, arg_scratch);
        if (tid == 0) out_tokens[row] = -last.index;
    } else if (tid == 0) {
        out_tokens[row] = found_index;
    }
}

}  // namespace

extern "C" long long mx_sample_scratch_bytes(int n_rows, int vocab) {
    return (long long)n_rows * vocab * (long long)sizeof(float);
}

extern "C" int mx_sample(const float* logits, long long row_stride, int n_rows, int vocab,
                         const float* temperature, const int* top_k, const float* top_p,
                         const float* repeat_penalty, const float* uniform,
                         const int* penalty_offsets, const int* penalty_ids, const int* pending_ids,
                         float* work, int* out_tokens, cudaStream_t stream) {
    if (n_rows <= 0) return MX_OK;
    if (vocab <= 0) MX_REFUSE("sample: vocabulary of %d", vocab);
    if (work == nullptr) MX_REFUSE("sample: needs a work buffer of rows x vocab floats");
    // greedy rows mark their penalised ids in a bitmap in shared memory, where the vocabulary fits in 32 KB of it
    const int words = (vocab + 31) / 32;
    const int mark_words = words * 4 <= 32 * 1024 ? words : 0;
    sample_kernel<<<n_rows, SAMPLE_THREADS, (size_t)mark_words * 4, stream>>>(
        logits, row_stride, vocab, temperature, top_k, top_p, repeat_penalty, uniform, penalty_offsets, penalty_ids,
        pending_ids, work, out_tokens, mark_words);
    return mx_launch_status();
}
