// Windowed attention with a softmax sink, and keys and values of different sizes.
//
//   q [n, H, dk], keys [.., G, dk], values [.., G, dv]; query head h reads kv head h / (H / G);
//   a query at absolute position a sees keys max(0, a + 1 - W) .. a (W = 0: all);
//   s_j = (q . k_j) * scale;  p_j = exp(s_j) / (sink + sum_i exp(s_i)),  sink = 1 or 0;  o = sum_j p_j v_j.
//
// The sink is a key of score 0 that has no value: it only takes its share of the weights.
//
// This file holds (1) the step between the q/k/v projection and attention: rotation of adjacent pairs
// (2i, 2i+1) of q and k by position, the mixing of this layer's values with those of an earlier layer, and the
// write of keys and values into their pages; (2) the fp32-arithmetic attention kernel for any sizes, one warp per
// (token, head), its keys in chunks of 32 aligned to absolute position so that a token's result depends on its own
// position and keys only.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------------------------
// rotation of pairs + value mixing + cache write
// ---------------------------------------------------------------------------------------------------------------
// qkv [n, H*dk + G*dk + G*dv] (bias already added).  Pair i < rot_dims/2 of every q and k head turns by the angle
// position * inv_freq[i], computed in fp32; dimensions from rot_dims on pass unchanged.
// mix_mode 0: values as they are; 1: also copy them to v_first (this layer is the source); 2: v = (1-lambda) v +
// lambda v_first.  What is cached is the mixed value.
template <typename T>
__global__ void qkv_pairs_post_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pages,
                                      T* __restrict__ v_pages, T* __restrict__ v_first, const float* __restrict__ inv_freq,
                                      const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
                                      const int32_t* __restrict__ block_table, int table_width, int page_size, int H, int G,
                                      int dk, int dv, int rot_dims, int mix_mode, float lambda) {
    const int t = blockIdx.x;
    const int pos = positions[t];
    const float fpos = (float)pos;
    const int width = (H + G) * dk + G * dv;
    const T* row = qkv + (size_t)t * width;
    long long page = -1;
    if (k_pages != nullptr) page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
    const int place = pos % page_size;
    const int half = (dk + 1) / 2;
    // q and k: one item per pair of adjacent dimensions
    for (int item = threadIdx.x; item < (H + G) * half; item += blockDim.x) {
        const int head = item / half, p = item - head * half;
        const int e0 = 2 * p, e1 = e0 + 1;
        float a = to_f32<T>(row[head * dk + e0]);
        float b = e1 < dk ? to_f32<T>(row[head * dk + e1]) : 0.0f;
        if (e1 < rot_dims) {
            float sn, cs;
            sincosf(fpos * inv_freq[p], &sn, &cs);
            const float ra = a * cs - b * sn, rb = b * cs + a * sn;
            a = ra;
            b = rb;
        }
        T* dst;
        if (head < H) {
            dst = q_out + ((size_t)t * H + head) * dk;
        } else {
            if (page < 0) continue;
            dst = k_pages + (((size_t)page * G + (head - H)) * page_size + place) * dk;
        }
        dst[e0] = from_f32<T>(a);
        if (e1 < dk) dst[e1] = from_f32<T>(b);
    }
    // v
    const T* vrow = row + (H + G) * dk;
    for (int item = threadIdx.x; item < G * dv; item += blockDim.x) {
        float v = to_f32<T>(vrow[item]);
        if (mix_mode == 1) v_first[(size_t)t * G * dv + item] = vrow[item];
        if (mix_mode == 2) v = (1.0f - lambda) * v + lambda * to_f32<T>(v_first[(size_t)t * G * dv + item]);
        if (page >= 0) {
            const int g = item / dv, e = item - g * dv;
            v_pages[(((size_t)page * G + g) * page_size + place) * dv + e] = from_f32<T>(v);
        }
    }
}

MM_EXPORT int mm_qkv_pairs_post(const void* qkv, void* q_out, void* k_pages, void* v_pages, void* v_first, int dtype,
                                const void* inv_freq, const void* positions, const void* token_req, const void* block_table,
                                int table_width, int page_size, int n_tokens, int H, int G, int dk, int dv, int rot_dims,
                                int mix_mode, float lambda, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && H > 0 && G > 0 && dk > 0 && dv > 0, "qkv post: bad sizes");
    MM_REQUIRE(rot_dims >= 0 && rot_dims <= dk && rot_dims % 2 == 0, "qkv post: the rotated dimensions must be even and at most the head size");
    MM_REQUIRE(mix_mode == 0 || v_first != nullptr, "qkv post: value mixing needs the first values");
    MM_REQUIRE(k_pages == nullptr || (page_size > 0 && table_width > 0 && v_pages != nullptr), "qkv post: bad page geometry");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 128;
    if (dtype == MM_F32)
        mm_launch(qkv_pairs_post_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)qkv, (float*)q_out, (float*)k_pages,
                  (float*)v_pages, (float*)v_first, (const float*)inv_freq, (const int32_t*)positions, (const int32_t*)token_req,
                  (const int32_t*)block_table, table_width, page_size, H, G, dk, dv, rot_dims, mix_mode, lambda);
    else if (dtype == MM_BF16)
        mm_launch(qkv_pairs_post_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, (const __nv_bfloat16*)qkv,
                  (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (__nv_bfloat16*)v_first,
                  (const float*)inv_freq, (const int32_t*)positions, (const int32_t*)token_req, (const int32_t*)block_table,
                  table_width, page_size, H, G, dk, dv, rot_dims, mix_mode, lambda);
    else
        MM_REQUIRE(false, "qkv post: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// attention, fp32 arithmetic, any sizes
// ---------------------------------------------------------------------------------------------------------------
#define SINK_MAX_ACC 16  // dv <= 512

template <typename T>
__global__ void attention_sink_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                                              const T* __restrict__ v_pages, T* __restrict__ out,
                                              const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
                                              const int32_t* __restrict__ block_table, int table_width, int page_size,
                                              int n_tokens, int H, int G, int dk, int dv, int window, float scale, int sink) {
    extern __shared__ float q_smem[];  // [warps][dk]
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * warps_per_block + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item - (long long)t * H);
    const int g = h / (H / G);
    const int pos = positions[t];
    const int32_t* table = block_table + (size_t)token_req[t] * table_width;
    const int hi = pos + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;

    float* qs = q_smem + warp * dk;
    const T* qrow = q + ((size_t)t * H + h) * dk;
    for (int d = lane; d < dk; d += 32) qs[d] = to_f32<T>(qrow[d]) * scale;
    __syncwarp();

    // the sink starts the running softmax: a maximum of 0 and a mass of 1 with nothing accumulated
    float m = sink ? 0.0f : -INFINITY, l = sink ? 1.0f : 0.0f;
    float acc[SINK_MAX_ACC];
#pragma unroll
    for (int a = 0; a < SINK_MAX_ACC; ++a) acc[a] = 0.0f;
    const size_t k_head = (size_t)g * page_size * dk, k_stride = (size_t)G * page_size * dk;
    const size_t v_head = (size_t)g * page_size * dv, v_stride = (size_t)G * page_size * dv;

    for (int c = (lo / 32) * 32; c < hi; c += 32) {
        const int j = c + lane;
        const bool valid = (j >= lo) && (j < hi);
        float s = -INFINITY;
        if (valid) {
            const int page = table[j / page_size];
            const T* kr = k_pages + (size_t)page * k_stride + k_head + (size_t)(j % page_size) * dk;
            float dot = 0.0f;
            for (int d = 0; d < dk; ++d) dot = fmaf(qs[d], to_f32<T>(kr[d]), dot);
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = expf(m - m_new);  // m = -inf on the first chunk gives 0
        const float p = valid ? expf(s - m_new) : 0.0f;
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int a = 0; a < SINK_MAX_ACC; ++a) acc[a] *= alpha;
        for (int jj = 0; jj < 32; ++jj) {
            const int key = c + jj;
            if (key < lo || key >= hi) continue;  // uniform over the warp
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int page = table[key / page_size];
            const T* vr = v_pages + (size_t)page * v_stride + v_head + (size_t)(key % page_size) * dv;
#pragma unroll
            for (int a = 0; a < SINK_MAX_ACC; ++a) {
                const int d = a * 32 + lane;
                if (d < dv) acc[a] = fmaf(pj, to_f32<T>(vr[d]), acc[a]);
            }
        }
        m = m_new;
    }
    const float inv_l = (l > 0.0f) ? 1.0f / l : 0.0f;
    T* orow = out + ((size_t)t * H + h) * dv;
#pragma unroll
    for (int a = 0; a < SINK_MAX_ACC; ++a) {
        const int d = a * 32 + lane;
        if (d < dv) orow[d] = from_f32<T>(acc[a] * inv_l);
    }
}

MM_EXPORT int mm_attention_sink_generic(const void* q, const void* k_pages, const void* v_pages, void* out, int dtype,
                                        const void* positions, const void* token_req, const void* block_table,
                                        int table_width, int page_size, int n_tokens, int H, int G, int dk, int dv, int window,
                                        float scale, int sink, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && H > 0 && G > 0 && dk > 0 && dv > 0 && H % G == 0, "attention: heads must be a positive multiple of kv heads");
    MM_REQUIRE(dv <= 32 * SINK_MAX_ACC && dk <= 2048, "attention: value size above 512 or key size above 2048 is not supported");
    MM_REQUIRE(page_size > 0 && table_width > 0 && window >= 0, "attention: bad page geometry or window");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = 4;
    const size_t smem = (size_t)warps * dk * sizeof(float);
    const long long items = (long long)n_tokens * H;
    const int blocks = (int)((items + warps - 1) / warps);
    if (dtype == MM_F32)
        mm_launch(attention_sink_generic_kernel<float>, dim3(blocks), dim3(warps * 32), smem, s, (const float*)q, (const float*)k_pages,
                  (const float*)v_pages, (float*)out, (const int32_t*)positions, (const int32_t*)token_req,
                  (const int32_t*)block_table, table_width, page_size, n_tokens, H, G, dk, dv, window, scale, sink);
    else if (dtype == MM_BF16)
        mm_launch(attention_sink_generic_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, s, (const __nv_bfloat16*)q,
                  (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out, (const int32_t*)positions,
                  (const int32_t*)token_req, (const int32_t*)block_table, table_width, page_size, n_tokens, H, G, dk, dv, window,
                  scale, sink);
    else
        MM_REQUIRE(false, "attention: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}
