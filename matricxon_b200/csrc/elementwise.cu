// Embedding lookup, LayerNorm, rotary encoding with the cache write, and the
// bias / activation / residual epilogue used behind a library matrix product.
//
// Formulas follow the reference's modules: token_embd lookup
// (app/architectures/starcoder2.py:218), nn.LayerNorm with biased variance
// (app/architectures/starcoder2_layers.py:45,56), NeoX rotate-half RoPE with fp32
// angles (app/architectures/rope.py:18-29,152-169; app/native/src/mx_fused_ops.c:20-34),
// K cached already rotated (app/architectures/qwen_layers.py:80-86), tanh GELU
// (app/architectures/starcoder2_layers.py:23).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

static thread_local char g_error[512] = "";
extern "C" const char* mx_last_error_message() { return g_error; }
// Programmatic dependent launch for the decode kernels: a kernel may start its preamble while the one
// before it drains. Measured on B200 inside CUDA graphs it makes a decode step of one or two rows
// faster (batch 1: 515 against 495 tokens/s) and a step of eight rows slower (2.27 against 2.18 ms), so
// the engine switches it per captured batch size with mx_set_chained_launch; MATRICXON_CHAINED_LAUNCH=0/1
// overrides that for every launch.
static int g_chained_launch = 0;
extern "C" void mx_set_chained_launch(int on) { g_chained_launch = on ? 1 : 0; }
bool mx_chained_launch_enabled() {
    static int forced = -2;
    if (forced == -2) {
        const char* value = getenv("MATRICXON_CHAINED_LAUNCH");
        forced = value == nullptr ? -1 : (value[0] == '1' ? 1 : 0);
    }
    return forced >= 0 ? forced == 1 : g_chained_launch == 1;
}

void mx_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ out, int hidden, int vocab, float scale, int* status) {
    pdl_trigger();
    const int row = blockIdx.x;
    const int id = ids[row];                 // step metadata: uploaded before the step, by no kernel
    float* o = out + (size_t)row * hidden;
    pdl_wait();
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, MX_STATUS_BAD_TOKEN_ID);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(src[i]) * scale;
}

// bfloat16 tables whose rows are a multiple of 8 wide: 16 bytes in, two float4 out per access.
__global__ void embed_vec_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab, float scale, int* status) {
    pdl_trigger();
    const int row = blockIdx.x;
    const int id = ids[row];
    float4* o = reinterpret_cast<float4*>(out + (size_t)row * hidden);
    pdl_wait();
    const int n_vec = hidden >> 3;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, MX_STATUS_BAD_TOKEN_ID);
        for (int i = threadIdx.x; i < 2 * n_vec; i += blockDim.x) o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * hidden);
    for (int i = threadIdx.x; i < n_vec; i += blockDim.x) {
        const uint4 v = __ldg(src + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        const float2 c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
        o[2 * i] = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
        o[2 * i + 1] = make_float4(c.x * scale, c.y * scale, d.x * scale, d.y * scale);
    }
}

// `scale` multiplies every looked-up value (1 for the architectures that take the table as it is).
extern "C" int mx_embed(const int* ids, const void* table, int dtype, float* out, int n_tokens,
                        int hidden, int vocab, float scale, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == MX_DTYPE_F32)
        mx_launch_chained(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, ids,
                          (const float*)table, out, hidden, vocab, scale, status);
    else if (hidden % 8 == 0 && (reinterpret_cast<uintptr_t>(table) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(out) & 15) == 0)
        mx_launch_chained(embed_vec_kernel, dim3(n_tokens), dim3(hidden >= 2048 ? 128 : 64), 0, stream, ids,
                          (const __nv_bfloat16*)table, out, hidden, vocab, scale, status);
    else
        mx_launch_chained(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, ids,
                          (const __nv_bfloat16*)table, out, hidden, vocab, scale, status);
    return mx_launch_status();
}

// logits <- cap * tanh(logits / cap), in place (float32): the soft cap some architectures put on
// their output scores.
__global__ void softcap_kernel(float* __restrict__ values, long long count, float cap) {
    pdl_trigger();
    pdl_wait();
    const float inv = 1.f / cap;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
        values[i] = cap * tanhf(values[i] * inv);
}

extern "C" int mx_softcap(float* values, long long count, float cap, cudaStream_t stream) {
    if (count <= 0) return MX_OK;
    if (!(cap > 0.f)) MX_REFUSE("softcap: the cap must be positive, not %f", (double)cap);
    const int blocks = (int)((count + 255) / 256 < 2048 ? (count + 255) / 256 : 2048);
    mx_launch_chained(softcap_kernel, dim3(blocks), dim3(256), 0, stream, values, count, cap);
    return mx_launch_status();
}

// ---------------------------------------------------------------- LayerNorm
// One block per output row. The row (float) is staged in shared memory; mean, then the
// mean of squared deviations (two passes, so no cancellation), all in float.
template <typename TOut>
__global__ void layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                 const float* __restrict__ weight, const float* __restrict__ bias,
                                 TOut* __restrict__ out, int hidden, float eps) {
    extern __shared__ float row_cache[];
    __shared__ float scratch[32];
    pdl_trigger();
    const int r = blockIdx.x;
    const int src_row = rows ? rows[r] : r;
    pdl_wait();
    const float* xr = after_wait(x) + (size_t)src_row * hidden;
    float s = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = xr[i];
        row_cache[i] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float q = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row_cache[i] - mean;
        q += d * d;
    }
    const float var = block_sum(q, scratch) / (float)hidden;
    const float rstd = 1.0f / sqrtf(var + eps);
    TOut* o = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = (row_cache[i] - mean) * rstd * weight[i];
        if (bias) v += bias[i];
        o[i] = from_float<TOut>(v);
    }
}

// The same for rows whose length is a multiple of 4 and at most 256 x 4 x LN_VPT: the row lives in
// registers as float4 vectors, read and written with 16-byte (8-byte for bfloat16) accesses.
constexpr int LN_VPT = 8;

template <typename TOut, int LN_THREADS>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_vec_kernel(const float* x, const int* __restrict__ rows,
                     const float* __restrict__ weight, const float* __restrict__ bias,
                     TOut* __restrict__ out, int hidden, float eps, const float* acc, const float* col_bias,
                     float* x_sum) {
    __shared__ float scratch[32];
    pdl_trigger();
    const int r = blockIdx.x;
    const int src_row = rows ? rows[r] : r;
    const int n_vec = hidden >> 2;
    const float4* w4 = reinterpret_cast<const float4*>(weight);
    const float4* b4 = reinterpret_cast<const float4*>(bias);
    // the norm's own constants are nobody's output: this thread's first vector of them sets out before the
    // wait on the kernel that writes x, instead of after the second reduction (a trip to L2 off the chain)
    float4 w_first = make_float4(0.f, 0.f, 0.f, 0.f), b_first = w_first;
    if ((int)threadIdx.x < n_vec) {
        w_first = w4[threadIdx.x];
        if (bias) b_first = b4[threadIdx.x];
    }
    pdl_wait();
    const float4* xr = reinterpret_cast<const float4*>(after_wait(x) + (size_t)src_row * hidden);
    float4 v[LN_VPT];
    float s = 0.f;
    if (acc != nullptr) {
        // the row is still a sum to be formed: x + (acc + col_bias), the residual epilogue of the product
        // before this norm (in that kernel's order of additions), written back to x on the way
        const float4* ar = reinterpret_cast<const float4*>(after_wait(acc) + (size_t)src_row * hidden);
        const float4* cb = reinterpret_cast<const float4*>(col_bias);
        float4* xw = reinterpret_cast<float4*>(after_wait(x_sum) + (size_t)src_row * hidden);
#pragma unroll
        for (int k = 0; k < LN_VPT; ++k) {
            const int i = threadIdx.x + k * LN_THREADS;
            v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < n_vec) {
                float4 a = ar[i];
                const float4 r = xr[i];
                if (col_bias) {
                    const float4 b = cb[i];
                    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
                }
                v[k] = make_float4(a.x + r.x, a.y + r.y, a.z + r.z, a.w + r.w);
                xw[i] = v[k];
            }
            s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        }
    } else {
#pragma unroll
        for (int k = 0; k < LN_VPT; ++k) {
            const int i = threadIdx.x + k * LN_THREADS;
            v[k] = i < n_vec ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        }
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < LN_VPT; ++k) {
        const int i = threadIdx.x + k * LN_THREADS;
        if (i < n_vec) {
            const float a = v[k].x - mean, b = v[k].y - mean, c = v[k].z - mean, d = v[k].w - mean;
            q += (a * a + b * b) + (c * c + d * d);
        }
    }
    const float var = block_sum(q, scratch) / (float)hidden;
    const float rstd = 1.0f / sqrtf(var + eps);
#pragma unroll
    for (int k = 0; k < LN_VPT; ++k) {
        const int i = threadIdx.x + k * LN_THREADS;
        if (i >= n_vec) continue;
        const float4 w = k == 0 ? w_first : w4[i];
        float4 y;
        y.x = (v[k].x - mean) * rstd * w.x; y.y = (v[k].y - mean) * rstd * w.y;
        y.z = (v[k].z - mean) * rstd * w.z; y.w = (v[k].w - mean) * rstd * w.w;
        if (bias) {
            const float4 b = k == 0 ? b_first : b4[i];
            y.x += b.x; y.y += b.y; y.z += b.z; y.w += b.w;
        }
        if (sizeof(TOut) == 4) {
            reinterpret_cast<float4*>(out + (size_t)r * hidden)[i] = y;
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
            uint2 packed;
            packed.x = *reinterpret_cast<unsigned*>(&lo);
            packed.y = *reinterpret_cast<unsigned*>(&hi);
            reinterpret_cast<uint2*>(out + (size_t)r * hidden)[i] = packed;
        }
    }
}

extern "C" int mx_epilogue(const void* acc, int acc_dtype, const float* bias, const float* residual, void* out,
                           int out_dtype, long long n_rows, int n_cols, int mode, cudaStream_t stream);

// acc != null: x (float, written) first becomes x + acc + col_bias (the residual epilogue of the product
// whose float accumulator acc is), in the same launch where the rows allow 16-byte accesses, else by the
// epilogue kernel ahead of the norm. rows must be null then.
static int layernorm_launch(float* x_sum, const float* x, const int* rows, const float* weight, const float* bias,
                            void* out, int out_dtype, int n_rows, int hidden, float eps, const float* acc,
                            const float* col_bias, cudaStream_t stream) {
    if (n_rows <= 0) return MX_OK;
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) |
                           reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(out) |
                           reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(col_bias)) & 15) == 0;
    if (hidden % 4 == 0 && hidden <= 4 * 256 * LN_VPT && aligned) {
        // about six vectors a thread: each thread then has six loads in flight, more blocks share an SM and
        // the two block-wide sums cross fewer warps (2,048 rows of 3,072: 9.8 us with 128 threads, 10.6
        // with 96, 12.4 with 256)
        // With few rows (decoding) the GPU is empty and the row's own latency is all there is: a thread per
        // vector where that fits (a decode step of 8 rows: 2.186 ms with 768 threads a row, 2.200 with 256,
        // 2.288 with 128).
        const int n_vec = hidden >> 2;
        int threads = ((n_vec + 5) / 6 + 31) / 32 * 32;
        threads = threads <= 64 ? 64 : (threads <= 96 ? 96 : (threads <= 128 ? 128 : (threads <= 192 ? 192 : 256)));
        if (n_rows <= 256) threads = n_vec <= 256 ? 256 : (n_vec <= 512 ? 512 : (n_vec <= 768 ? 768 : 1024));
#define MX_LN_LAUNCH(T, N)                                                                                       \
    mx_launch_chained(layernorm_vec_kernel<T, N>, dim3(n_rows), dim3(N), 0, stream, x, rows, weight, bias, (T*)out, \
                      hidden, eps, acc, col_bias, x_sum)
        if (out_dtype == MX_DTYPE_F32) {
            if (threads == 64) MX_LN_LAUNCH(float, 64);
            else if (threads == 96) MX_LN_LAUNCH(float, 96);
            else if (threads == 128) MX_LN_LAUNCH(float, 128);
            else if (threads == 192) MX_LN_LAUNCH(float, 192);
            else if (threads == 512) MX_LN_LAUNCH(float, 512);
            else if (threads == 768) MX_LN_LAUNCH(float, 768);
            else if (threads == 1024) MX_LN_LAUNCH(float, 1024);
            else MX_LN_LAUNCH(float, 256);
        } else {
            if (threads == 64) MX_LN_LAUNCH(__nv_bfloat16, 64);
            else if (threads == 96) MX_LN_LAUNCH(__nv_bfloat16, 96);
            else if (threads == 128) MX_LN_LAUNCH(__nv_bfloat16, 128);
            else if (threads == 192) MX_LN_LAUNCH(__nv_bfloat16, 192);
            else if (threads == 512) MX_LN_LAUNCH(__nv_bfloat16, 512);
            else if (threads == 768) MX_LN_LAUNCH(__nv_bfloat16, 768);
            else if (threads == 1024) MX_LN_LAUNCH(__nv_bfloat16, 1024);
            else MX_LN_LAUNCH(__nv_bfloat16, 256);
        }
#undef MX_LN_LAUNCH
        return mx_launch_status();
    }
    if (acc != nullptr) {       // the general kernel takes a finished row: the sum is formed by the epilogue kernel
        const int rc = mx_epilogue(acc, MX_DTYPE_F32, col_bias, x, x_sum, MX_DTYPE_F32, n_rows, hidden, 2, stream);
        if (rc != MX_OK) return rc;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) MX_REFUSE("layernorm: hidden size %d exceeds the 51200 this kernel stages", hidden);
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (out_dtype == MX_DTYPE_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mx_launch_chained(layernorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, rows, weight,
                          bias, (float*)out, hidden, eps);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(layernorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mx_launch_chained(layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream, x, rows,
                          weight, bias, (__nv_bfloat16*)out, hidden, eps);
    }
    return mx_launch_status();
}

extern "C" int mx_layernorm(const float* x, const int* rows, const float* weight, const float* bias,
                            void* out, int out_dtype, int n_rows, int hidden, float eps,
                            cudaStream_t stream) {
    return layernorm_launch(nullptr, x, rows, weight, bias, out, out_dtype, n_rows, hidden, eps, nullptr, nullptr,
                            stream);
}

// x <- x + acc + col_bias (col_bias may be null), then out <- LayerNorm(x): the residual epilogue of a
// product and the norm after it in one pass over the rows.
extern "C" int mx_layernorm_sum(float* x, const float* acc, const float* col_bias, const float* weight,
                                const float* bias, void* out, int out_dtype, int n_rows, int hidden, float eps,
                                cudaStream_t stream) {
    if (acc == nullptr) MX_REFUSE("layernorm with sum: no accumulator");
    return layernorm_launch(x, x, nullptr, weight, bias, out, out_dtype, n_rows, hidden, eps, acc, col_bias, stream);
}

// ---------------------------------------------------------------- rotary + cache write
// qkv rows are [q heads | k heads | v heads], each head `head_dim` wide. q is rotated in
// place; k is rotated and stored, v is stored, at `slot = page * page_size + offset` of a
// cache laid out [page][2 (k,v)][kv head][page_size x head_dim], keys as [slot][dim] and values
// transposed as [dim][slot] (so a tensor-core B operand reads keys contiguously). Angles and the rotation
// are float; one rounding to T at the end. With write_cache == 0 only q is rotated. A slot of
// -1 marks a padding row (rotated, not stored); any other slot outside the pool sets the
// status bit MX_STATUS_BAD_SLOT.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride,
                                     const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq,
                                     const int* __restrict__ slots, T* __restrict__ cache,
                                     int n_heads, int n_kv_heads, int head_dim, int rotary_dim,
                                     int page_size, long long n_slots, int write_cache,
                                     int* status, const float* __restrict__ col_bias) {
    extern __shared__ float cs[];  // cos[half], sin[half]
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = rotary_dim >> 1;
    const float pos = (float)positions[t];   // step metadata and constants: no kernel writes them
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float angle = pos * inv_freq[i];
        cs[i] = cosf(angle);
        cs[half + i] = sinf(angle);
    }
    __syncthreads();
    pdl_wait();
    T* row = after_wait(qkv) + (size_t)t * row_stride;
    // col_bias: the product's bias, still to be added (the product came from the library without an
    // epilogue). The sum is rounded to T first, as the epilogue kernel would have left it.
    auto value = [&](const T* p, int col) {
        return col_bias ? to_float(from_float<T>(to_float(*p) + col_bias[col])) : to_float(*p);
    };

    // q heads: rotate in place
    for (int item = threadIdx.x; item < n_heads * half; item += blockDim.x) {
        const int h = item / half, i = item - h * half;
        T* p = row + (size_t)h * head_dim;
        const float x1 = value(p + i, h * head_dim + i), x2 = value(p + i + half, h * head_dim + i + half);
        const float c = cs[i], s = cs[half + i];
        p[i] = from_float<T>(x1 * c - x2 * s);
        p[i + half] = from_float<T>(x2 * c + x1 * s);
    }
    if (col_bias)                                 // q dims beyond the rotary width still want their bias
        for (int item = threadIdx.x; item < n_heads * (head_dim - rotary_dim); item += blockDim.x) {
            const int h = item / (head_dim - rotary_dim), i = rotary_dim + item - h * (head_dim - rotary_dim);
            T* p = row + (size_t)h * head_dim + i;
            *p = from_float<T>(value(p, h * head_dim + i));
        }
    if (!write_cache) return;

    const long long slot = slots[t];
    if (slot == -1) return;  // a padding row of a fixed-size batch: nothing to store
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(status, MX_STATUS_BAD_SLOT);
        return;
    }
    const long long page = slot / page_size;
    const int offset = (int)(slot - page * page_size);
    const size_t head_stride = (size_t)page_size * head_dim;
    // keys: [page][0][kv head][slot][dim]; values transposed: [page][1][kv head][dim][slot]
    T* kbase = cache + ((size_t)page * 2 * n_kv_heads) * head_stride + (size_t)offset * head_dim;
    T* vbase = cache + ((size_t)page * 2 * n_kv_heads + n_kv_heads) * head_stride + offset;
    const T* krow = row + (size_t)n_heads * head_dim;
    const T* vrow = krow + (size_t)n_kv_heads * head_dim;

    const int kcol = n_heads * head_dim, vcol = (n_heads + n_kv_heads) * head_dim;
    for (int item = threadIdx.x; item < n_kv_heads * half; item += blockDim.x) {
        const int h = item / half, i = item - h * half;
        const T* p = krow + (size_t)h * head_dim;
        const float x1 = value(p + i, kcol + h * head_dim + i), x2 = value(p + i + half, kcol + h * head_dim + i + half);
        const float c = cs[i], s = cs[half + i];
        T* dst = kbase + (size_t)h * head_stride;
        dst[i] = from_float<T>(x1 * c - x2 * s);
        dst[i + half] = from_float<T>(x2 * c + x1 * s);
    }
    // dims beyond the rotary width pass through unrotated
    const int tail = head_dim - rotary_dim;
    for (int item = threadIdx.x; item < n_kv_heads * tail; item += blockDim.x) {
        const int h = item / tail, i = rotary_dim + (item - h * tail);
        kbase[(size_t)h * head_stride + i] = from_float<T>(value(krow + (size_t)h * head_dim + i, kcol + h * head_dim + i));
    }
    for (int item = threadIdx.x; item < n_kv_heads * head_dim; item += blockDim.x) {
        const int h = item / head_dim, i = item - h * head_dim;
        vbase[(size_t)h * head_stride + (size_t)i * page_size] =
            from_float<T>(value(vrow + (size_t)h * head_dim + i, vcol + h * head_dim + i));
    }
}

// The same with 16-byte accesses: each thread rotates E consecutive pairs (E = 8 for bfloat16,
// 4 for float). Needs rotary_dim / 2, head_dim and the row stride to be multiples of E.
template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, int row_stride,
                                         const int* __restrict__ positions,
                                         const float* __restrict__ inv_freq,
                                         const int* __restrict__ slots, T* __restrict__ cache,
                                         int n_heads, int n_kv_heads, int head_dim, int rotary_dim,
                                         int page_size, long long n_slots, int write_cache,
                                         int* status, const float* __restrict__ col_bias) {
    constexpr int E = 16 / sizeof(T);
    extern __shared__ float cs[];  // cos[half], sin[half]
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = rotary_dim >> 1;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float angle = pos * inv_freq[i];
        cs[i] = cosf(angle);
        cs[half + i] = sinf(angle);
    }
    __syncthreads();
    pdl_wait();
    T* row = after_wait(qkv) + (size_t)t * row_stride;
    const int per_head = half / E;
    // col_bias: see rope_kv_write_kernel
    auto value = [&](T v, int col) {
        return col_bias ? to_float(from_float<T>(to_float(v) + col_bias[col])) : to_float(v);
    };

    long long slot = -1;
    if (write_cache) {
        slot = slots[t];
        if (slot != -1 && (slot < 0 || slot >= n_slots)) {
            if (threadIdx.x == 0) atomicOr(status, MX_STATUS_BAD_SLOT);
            slot = -1;
        }
    }
    const long long page = slot >= 0 ? slot / page_size : 0;
    const int offset = slot >= 0 ? (int)(slot - page * page_size) : 0;
    const size_t head_stride = (size_t)page_size * head_dim;
    T* kbase = cache + ((size_t)page * 2 * n_kv_heads) * head_stride + (size_t)offset * head_dim;
    T* vbase = cache + ((size_t)page * 2 * n_kv_heads + n_kv_heads) * head_stride + offset;

    // q heads (in place) and k heads (into the cache), E pairs per thread
    const int rot_heads = n_heads + (slot >= 0 ? n_kv_heads : 0);
    for (int item = threadIdx.x; item < rot_heads * per_head; item += blockDim.x) {
        const int h = item / per_head, i = (item - h * per_head) * E;
        const T* src = row + (size_t)h * head_dim;
        uint4 lo_raw = *reinterpret_cast<const uint4*>(src + i);
        uint4 hi_raw = *reinterpret_cast<const uint4*>(src + i + half);
        T* lo = reinterpret_cast<T*>(&lo_raw);
        T* hi = reinterpret_cast<T*>(&hi_raw);
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float x1 = value(lo[e], h * head_dim + i + e), x2 = value(hi[e], h * head_dim + i + half + e);
            const float c = cs[i + e], sn = cs[half + i + e];
            lo[e] = from_float<T>(x1 * c - x2 * sn);
            hi[e] = from_float<T>(x2 * c + x1 * sn);
        }
        T* dst = h < n_heads ? row + (size_t)h * head_dim
                             : kbase + (size_t)(h - n_heads) * head_stride;
        *reinterpret_cast<uint4*>(dst + i) = lo_raw;
        *reinterpret_cast<uint4*>(dst + i + half) = hi_raw;
    }
    const int tail = head_dim - rotary_dim;          // dims beyond the rotary width pass through
    if (col_bias)                                    // ... with their bias, for q in place
        for (int item = threadIdx.x; item < n_heads * tail; item += blockDim.x) {
            const int h = item / tail, i = rotary_dim + (item - h * tail);
            T* p = row + (size_t)h * head_dim + i;
            *p = from_float<T>(value(*p, h * head_dim + i));
        }
    if (slot < 0) return;
    const T* krow = row + (size_t)n_heads * head_dim;
    const T* vrow = krow + (size_t)n_kv_heads * head_dim;
    const int kcol = n_heads * head_dim, vcol = (n_heads + n_kv_heads) * head_dim;
    for (int item = threadIdx.x; item < n_kv_heads * tail; item += blockDim.x) {
        const int h = item / tail, i = rotary_dim + (item - h * tail);
        kbase[(size_t)h * head_stride + i] = from_float<T>(value(krow[(size_t)h * head_dim + i], kcol + h * head_dim + i));
    }
    for (int item = threadIdx.x; item < n_kv_heads * head_dim; item += blockDim.x) {
        const int h = item / head_dim, i = item - h * head_dim;
        vbase[(size_t)h * head_stride + (size_t)i * page_size] =
            from_float<T>(value(vrow[(size_t)h * head_dim + i], vcol + h * head_dim + i));
    }
}

// col_bias (may be null): the bias of the product that made qkv, when that product ran without its epilogue
// (the library's, for 17 or more rows): it is added here, rounded as the epilogue would have rounded it,
// and the epilogue's pass over qkv is saved.
extern "C" int mx_rope_kv_write_bias(void* qkv, int dtype, int row_stride, const int* positions,
                                const float* inv_freq, const int* slots, void* cache, int n_tokens,
                                int n_heads, int n_kv_heads, int head_dim, int rotary_dim,
                                int page_size, long long n_pages, int write_cache, int* status,
                                const float* col_bias, cudaStream_t stream) {
    if (n_tokens <= 0) return MX_OK;
    if (rotary_dim % 2 != 0 || rotary_dim > head_dim || rotary_dim < 0)
        MX_REFUSE("rope: rotary width %d must be even and at most head_dim %d", rotary_dim, head_dim);
    const size_t smem = (size_t)rotary_dim * sizeof(float);
    if (smem > 48 * 1024) MX_REFUSE("rope: rotary width %d is too large", rotary_dim);
    const int work = n_heads * (rotary_dim / 2);
    const int threads = work >= 1024 ? 256 : 128;
    const long long n_slots = n_pages * page_size;
    const int lanes = dtype == MX_DTYPE_F32 ? 4 : 8;
    const bool vec = rotary_dim > 0 && (rotary_dim / 2) % lanes == 0 && head_dim % lanes == 0 &&
                     row_stride % lanes == 0 && (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(cache) & 15) == 0;
    if (vec) {
        if (dtype == MX_DTYPE_F32)
            mx_launch_chained(rope_kv_write_vec_kernel<float>, dim3(n_tokens), dim3(threads), smem, stream,
                              (float*)qkv, row_stride, positions, inv_freq, slots, (float*)cache, n_heads,
                              n_kv_heads, head_dim, rotary_dim, page_size, n_slots, write_cache, status, col_bias);
        else
            mx_launch_chained(rope_kv_write_vec_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), smem,
                              stream, (__nv_bfloat16*)qkv, row_stride, positions, inv_freq, slots,
                              (__nv_bfloat16*)cache, n_heads, n_kv_heads, head_dim, rotary_dim, page_size,
                              n_slots, write_cache, status, col_bias);
        return mx_launch_status();
    }
    if (dtype == MX_DTYPE_F32)
        mx_launch_chained(rope_kv_write_kernel<float>, dim3(n_tokens), dim3(threads), smem, stream,
                          (float*)qkv, row_stride, positions, inv_freq, slots, (float*)cache, n_heads,
                          n_kv_heads, head_dim, rotary_dim, page_size, n_slots, write_cache, status, col_bias);
    else
        mx_launch_chained(rope_kv_write_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), smem, stream,
                          (__nv_bfloat16*)qkv, row_stride, positions, inv_freq, slots,
                          (__nv_bfloat16*)cache, n_heads, n_kv_heads, head_dim, rotary_dim, page_size,
                          n_slots, write_cache, status, col_bias);
    return mx_launch_status();
}

extern "C" int mx_rope_kv_write(void* qkv, int dtype, int row_stride, const int* positions,
                                const float* inv_freq, const int* slots, void* cache, int n_tokens,
                                int n_heads, int n_kv_heads, int head_dim, int rotary_dim,
                                int page_size, long long n_pages, int write_cache, int* status,
                                cudaStream_t stream) {
    return mx_rope_kv_write_bias(qkv, dtype, row_stride, positions, inv_freq, slots, cache, n_tokens, n_heads, n_kv_heads,
                                 head_dim, rotary_dim, page_size, n_pages, write_cache, status, nullptr, stream);
}

// ---------------------------------------------------------------- epilogue behind a library GEMM
// mode 0: out(T)  = acc + bias
// mode 1: out(T)  = gelu_tanh(acc + bias)
// mode 2: out(f32) = residual + acc + bias     (out may alias residual)
// mode 3: out(f32) = acc + bias
template <typename TAcc, typename TOut>
__global__ void epilogue_kernel(const TAcc* __restrict__ acc, const float* __restrict__ bias,
                                const float* residual, TOut* out, long long total, int n_cols,
                                int mode) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        float v = to_float(acc[i]);
        if (bias) v += bias[(int)(i % n_cols)];
        if (mode == 1) v = gelu_tanh(v);
        if (mode == 2) v += residual[i];
        out[i] = from_float<TOut>(v);
    }
}

// The same, four neighbouring columns per item (rows whose length is a multiple of 4, 16-byte aligned
// tensors, fewer than 2^31 elements) and EPI_ITEMS items per thread, a grid apart: every item's loads are
// issued before the first is used, so that a thread has 64 to 128 bytes on their way instead of 8 to 32
// (the first product of the feed-forward at 256 rows: 7.7 us with one item a thread).
constexpr int EPI_ITEMS = 4;
template <typename TAcc, typename TOut>
__global__ void epilogue_vec_kernel(const TAcc* __restrict__ acc, const float* __restrict__ bias,
                                    const float* residual, TOut* out, int total4, int cols4, int mode) {
    const int first = blockIdx.x * blockDim.x + threadIdx.x, stride = gridDim.x * blockDim.x;
    float v[EPI_ITEMS][4];
    float4 r[EPI_ITEMS], b[EPI_ITEMS];
#pragma unroll
    for (int k = 0; k < EPI_ITEMS; ++k) {
        const int i4 = first + k * stride;
        if (i4 >= total4) continue;
        const size_t at = (size_t)i4 * 4;
        if (sizeof(TAcc) == 4) {
            const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(acc) + at);
            v[k][0] = a.x; v[k][1] = a.y; v[k][2] = a.z; v[k][3] = a.w;
        } else {
            const uint2 a = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(acc) + at);
            const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&a.x);
            const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&a.y);
            v[k][0] = __low2float(lo); v[k][1] = __high2float(lo); v[k][2] = __low2float(hi); v[k][3] = __high2float(hi);
        }
        if (bias) b[k] = __ldg(reinterpret_cast<const float4*>(bias + (i4 % cols4) * 4));
        if (mode == 2) r[k] = *reinterpret_cast<const float4*>(residual + at);
    }
#pragma unroll
    for (int k = 0; k < EPI_ITEMS; ++k) {
        const int i4 = first + k * stride;
        if (i4 >= total4) continue;
        const size_t at = (size_t)i4 * 4;
        if (bias) { v[k][0] += b[k].x; v[k][1] += b[k].y; v[k][2] += b[k].z; v[k][3] += b[k].w; }
        if (mode == 1) {
            // a result that is rounded to bfloat16 takes the hardware tanh, as in the engine's own products
#pragma unroll
            for (int e = 0; e < 4; ++e) v[k][e] = sizeof(TOut) == 4 ? gelu_tanh(v[k][e]) : gelu_tanh_fast(v[k][e]);
        }
        if (mode == 2) { v[k][0] += r[k].x; v[k][1] += r[k].y; v[k][2] += r[k].z; v[k][3] += r[k].w; }
        if (sizeof(TOut) == 4) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + at) = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(v[k][0], v[k][1]), hi = __floats2bfloat162_rn(v[k][2], v[k][3]);
            uint2 packed;
            packed.x = *reinterpret_cast<unsigned*>(&lo);
            packed.y = *reinterpret_cast<unsigned*>(&hi);
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + at) = packed;
        }
    }
}

extern "C" int mx_epilogue(const void* acc, int acc_dtype, const float* bias, const float* residual,
                           void* out, int out_dtype, long long n_rows, int n_cols, int mode,
                           cudaStream_t stream) {
    const long long total = n_rows * n_cols;
    if (total <= 0) return MX_OK;
    if (mode < 0 || mode > 3) MX_REFUSE("epilogue: unknown mode %d", mode);
    if (mode == 2 && residual == nullptr) MX_REFUSE("epilogue: residual mode without a residual");
    const int threads = 256;
    const bool aligned = ((reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(bias) |
                           reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (n_cols % 4 == 0 && aligned && total < (1LL << 31)) {
        const int total4 = (int)(total / 4), cols4 = n_cols / 4;
        const int vblocks = (total4 + threads * EPI_ITEMS - 1) / (threads * EPI_ITEMS);
#define MX_EPI_VEC(TA, TO) \
    epilogue_vec_kernel<TA, TO><<<vblocks, threads, 0, stream>>>((const TA*)acc, bias, residual, (TO*)out, total4, cols4, mode)
        if (acc_dtype == MX_DTYPE_F32 && out_dtype == MX_DTYPE_F32) MX_EPI_VEC(float, float);
        else if (acc_dtype == MX_DTYPE_F32) MX_EPI_VEC(float, __nv_bfloat16);
        else if (out_dtype == MX_DTYPE_F32) MX_EPI_VEC(__nv_bfloat16, float);
        else MX_EPI_VEC(__nv_bfloat16, __nv_bfloat16);
#undef MX_EPI_VEC
        return mx_launch_status();
    }
    long long blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
#define MX_EPI(TA, TO) \
    epilogue_kernel<TA, TO><<<(int)blocks, threads, 0, stream>>>((const TA*)acc, bias, residual, (TO*)out, total, n_cols, mode)
    if (acc_dtype == MX_DTYPE_F32 && out_dtype == MX_DTYPE_F32) MX_EPI(float, float);
    else if (acc_dtype == MX_DTYPE_F32) MX_EPI(float, __nv_bfloat16);
    else if (out_dtype == MX_DTYPE_F32) MX_EPI(__nv_bfloat16, float);
    else MX_EPI(__nv_bfloat16, __nv_bfloat16);
#undef MX_EPI
    return mx_launch_status();
}
