// Token embedding plus a hashed embedding of the pair (previous token, token).
//
//   x[t] = E[id_t] + B[row_t],   row_t = (prev_t * mul_prev + id_t * mul_cur) mod buckets,
//   row_t = buckets (the table's extra last row) for the first token of a sequence (position 0).
//
// The previous token of a portion's first token is not in the step: it is per-request state, one int32 per state
// slot.  The block of a request's first token in the step reads the state and then (the same thread, so the order
// is fixed) stores the request's last token of this step for the next one.  Requests with one token each
// (`req_meta` null: a decode batch) are their own first and last token.
#include "common.cuh"

template <typename T>
__global__ void embedding_bigram_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ positions,
                                        const int32_t* __restrict__ token_req, const int32_t* __restrict__ req_meta,
                                        const int32_t* __restrict__ slots, int32_t* __restrict__ state,
                                        const T* __restrict__ table, const T* __restrict__ pairs, float* __restrict__ out,
                                        int vocab, int d, int buckets, long long mul_prev, long long mul_cur) {
    __shared__ int s_prev;
    const int t = blockIdx.x;
    const int id = ids[t];
    if (threadIdx.x == 0) {
        const int r = token_req[t];
        const bool first = (t == 0) || (token_req[t - 1] != r);
        int prev = -1;
        if (positions[t] > 0) prev = first ? state[slots[r]] : ids[t - 1];
        if (first) {
            const int last = req_meta ? req_meta[4 * r] + req_meta[4 * r + 1] - 1 : t;
            state[slots[r]] = ids[last];
        }
        s_prev = prev;
    }
    __syncthreads();
    const int prev = s_prev;
    float* o = out + (size_t)t * d;
    if (id < 0 || id >= vocab) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    long long row = buckets;
    if (prev >= 0) {
        row = ((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets;
        if (row < 0) row += buckets;
    }
    const T* e = table + (size_t)id * d;
    const T* b = pairs + (size_t)row * d;
    if (sizeof(T) == 2 && d % 8 == 0 && (((uintptr_t)table | (uintptr_t)pairs | (uintptr_t)out) & 15) == 0) {
        // bfloat16 rows of a multiple of 8: one 16-byte load of each table and two 16-byte stores per thread and step
        for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
            const uint4 ra = *reinterpret_cast<const uint4*>(e + i), rb = *reinterpret_cast<const uint4*>(b + i);
            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&ra);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&rb);
            float f[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 x = __bfloat1622float2(a2[k]), y = __bfloat1622float2(b2[k]);
                f[2 * k] = x.x + y.x;
                f[2 * k + 1] = x.y + y.y;
            }
            *reinterpret_cast<float4*>(o + i) = make_float4(f[0], f[1], f[2], f[3]);
            *reinterpret_cast<float4*>(o + i + 4) = make_float4(f[4], f[5], f[6], f[7]);
        }
        return;
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f32<T>(e[i]) + to_f32<T>(b[i]);
}

MM_EXPORT int mm_embedding_bigram(const void* ids, const void* positions, const void* token_req, const void* req_meta,
                                  const void* slots, void* state, const void* table, const void* pairs, int dtype, void* out,
                                  int n_tokens, int vocab, int d, int buckets, long long mul_prev, long long mul_cur, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && vocab > 0 && d > 0 && buckets > 0, "bigram embedding: bad sizes");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (dtype == MM_F32)
        mm_launch(embedding_bigram_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const int32_t*)ids, (const int32_t*)positions,
                  (const int32_t*)token_req, (const int32_t*)req_meta, (const int32_t*)slots, (int32_t*)state, (const float*)table,
                  (const float*)pairs, (float*)out, vocab, d, buckets, mul_prev, mul_cur);
    else if (dtype == MM_BF16)
        mm_launch(embedding_bigram_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, (const int32_t*)ids,
                  (const int32_t*)positions, (const int32_t*)token_req, (const int32_t*)req_meta, (const int32_t*)slots,
                  (int32_t*)state, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs, (float*)out, vocab, d, buckets,
                  mul_prev, mul_cur);
    else
        MM_REQUIRE(false, "bigram embedding: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}
