// minGRU: a gated recurrence whose gates read only the current token, so that a prompt is a linear scan.
//
//   z = sigmoid(a_z),  c = a_x + 1/2 where a_x >= 0, sigmoid(a_x) below,
//   S_t = (1 - z) S_(t-1) + z c      (element by element, fp32, state carried per request)
//   y_t = S_t * silu(a_g)
//
// a = [a_z | a_x | a_g] is the fp32 output of one projection, [n, 3W]; the biases of the gate and the candidate
// (bias [2W] fp32, or null) are added here.  Everything here is fp32; y is written in the activation dtype for the
// output projection.  The loads of a token do not depend on the recurrence: the loops fetch MG_AHEAD tokens at a time.
//
// Two routes.  Few tokens per request: one thread per (request, channel) walks the request's tokens.  Long portions:
// the tokens are cut into chunks; every chunk is scanned from a zero state and gives the pair (A, B) with
// S_end = A S_start + B; a second pass walks the chunks of a request in order and leaves every chunk's starting
// state; a third pass scans every chunk again from its starting state and writes y.  The state a request starts
// from is its slot's, or zero at position 0 whatever the slot still holds.
#include "common.cuh"

#define MG_AHEAD 8

// FAST: the hardware's exponential and reciprocal (about 2 units in the last place of fp32) for bfloat16 runs, whose
// outputs are rounded to 8 bits anyway: with the exact functions the scan is bound by instructions (two exponentials
// and two IEEE divisions per token and channel), not by memory.  float32 runs take the exact ones.
template <bool FAST>
__device__ __forceinline__ float sigmoid_f32(float x) {
    return FAST ? __fdividef(1.0f, 1.0f + __expf(-x)) : 1.0f / (1.0f + expf(-x));
}

template <bool FAST>
__device__ __forceinline__ void mingru_gate(float az, float ax, float& keep, float& add) {
    const float z = sigmoid_f32<FAST>(az);
    const float c = ax >= 0.0f ? ax + 0.5f : sigmoid_f32<FAST>(ax);
    keep = 1.0f - z;
    add = z * c;
}

// n tokens from t0 on for channel c, starting from the state S; WRITE: y gets state * silu(gate); prod (if given)
// gets the product of the keep factors.  Returns the last state.
template <typename T, bool WRITE, bool FAST>
__device__ __forceinline__ float mingru_run(const float* __restrict__ a, T* __restrict__ y, int t0, int n, int c, int W, float bz,
                                            float bx, float S, float* prod) {
    float p = 1.0f;
    for (int t = t0; t < t0 + n; t += MG_AHEAD) {
        float az[MG_AHEAD], ax[MG_AHEAD], ag[MG_AHEAD];
#pragma unroll
        for (int k = 0; k < MG_AHEAD; ++k) {
            const bool in = t + k < t0 + n;
            const float* row = a + (size_t)(in ? t + k : t) * 3 * W;
            az[k] = row[c];
            ax[k] = row[W + c];
            ag[k] = WRITE ? row[2 * W + c] : 0.0f;
        }
#pragma unroll
        for (int k = 0; k < MG_AHEAD; ++k) {
            if (t + k < t0 + n) {
                float keep, add;
                mingru_gate<FAST>(az[k] + bz, ax[k] + bx, keep, add);
                S = fmaf(keep, S, add);
                p *= keep;
                if (WRITE) y[(size_t)(t + k) * W + c] = from_f32<T>(S * (ag[k] * sigmoid_f32<FAST>(ag[k])));
            }
        }
    }
    if (prod) *prod = p;
    return S;
}

// req_meta [requests, 4] = (first token, tokens, ., .) or null: every request is one token, request r is token r
template <typename T>
__global__ void mingru_walk_kernel(const float* __restrict__ a, T* __restrict__ y, float* __restrict__ state,
                                   const int32_t* __restrict__ req_meta, const int32_t* __restrict__ slots,
                                   const int32_t* __restrict__ positions, const float* __restrict__ bias, int W) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= W) return;
    const int t0 = req_meta ? req_meta[4 * r] : r;
    const int n = req_meta ? req_meta[4 * r + 1] : 1;
    float* st = state + (size_t)slots[r] * W + c;
    float S = positions[t0] == 0 ? 0.0f : *st;
    const float bz = bias ? bias[c] : 0.0f, bx = bias ? bias[W + c] : 0.0f;
    S = mingru_run<T, true, sizeof(T) == 2>(a, y, t0, n, c, W, bz, bx, S, nullptr);
    *st = S;
}

// pass 1: chunk k of request r (tokens t0 + k*chunk ...) from a zero state -> A[ck], B[ck]
template <bool FAST>
__global__ void mingru_chunk_reduce_kernel(const float* __restrict__ a, float* __restrict__ A, float* __restrict__ B,
                                           const int32_t* __restrict__ chunk_meta, const float* __restrict__ bias, int W) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int ck = blockIdx.y;
    if (c >= W) return;
    const int t0 = chunk_meta[4 * ck], n = chunk_meta[4 * ck + 1];
    const float bz = bias ? bias[c] : 0.0f, bx = bias ? bias[W + c] : 0.0f;
    float prod;
    const float S = mingru_run<float, false, FAST>(a, nullptr, t0, n, c, W, bz, bx, 0.0f, &prod);
    A[(size_t)ck * W + c] = prod;
    B[(size_t)ck * W + c] = S;
}

// pass 2: per request, in chunk order: B[ck] <- the state the chunk starts from; the slot gets the final state.
// chunk_meta [chunks, 4] = (first token, tokens, request, first chunk of the request ? 1 : 0); req_chunks [requests, 2]
// = (first chunk, chunks).
__global__ void mingru_chunk_carry_kernel(const float* __restrict__ A, float* __restrict__ B, float* __restrict__ state,
                                          const int32_t* __restrict__ req_chunks, const int32_t* __restrict__ chunk_meta,
                                          const int32_t* __restrict__ slots, const int32_t* __restrict__ positions, int W) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= W) return;
    const int k0 = req_chunks[2 * r], nk = req_chunks[2 * r + 1];
    if (nk == 0) return;
    float* st = state + (size_t)slots[r] * W + c;
    float S = positions[chunk_meta[4 * k0]] == 0 ? 0.0f : *st;
    for (int k = k0; k < k0 + nk; ++k) {
        const size_t i = (size_t)k * W + c;
        const float start = S;
        S = fmaf(A[i], S, B[i]);
        B[i] = start;
    }
    *st = S;
}

// pass 3: every chunk again from its starting state, writing y
template <typename T>
__global__ void mingru_chunk_apply_kernel(const float* __restrict__ a, const float* __restrict__ start, T* __restrict__ y,
                                          const int32_t* __restrict__ chunk_meta, const float* __restrict__ bias, int W) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int ck = blockIdx.y;
    if (c >= W) return;
    const int t0 = chunk_meta[4 * ck], n = chunk_meta[4 * ck + 1];
    const float bz = bias ? bias[c] : 0.0f, bx = bias ? bias[W + c] : 0.0f;
    mingru_run<T, true, sizeof(T) == 2>(a, y, t0, n, c, W, bz, bx, start[(size_t)ck * W + c], nullptr);
}

MM_EXPORT int mm_mingru_walk(const void* a, void* y, int dtype, void* state, const void* req_meta, const void* slots,
                             const void* positions, const void* bias, int n_requests, int W, void* stream) {
    MM_REQUIRE(n_requests >= 0 && W > 0, "mingru: bad sizes");
    if (n_requests == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = W >= 128 ? 128 : 64;
    dim3 grid(ceil_div(W, threads), n_requests);
    if (dtype == MM_F32)
        mm_launch(mingru_walk_kernel<float>, grid, dim3(threads), 0, s, (const float*)a, (float*)y, (float*)state,
                  (const int32_t*)req_meta, (const int32_t*)slots, (const int32_t*)positions, (const float*)bias, W);
    else if (dtype == MM_BF16)
        mm_launch(mingru_walk_kernel<__nv_bfloat16>, grid, dim3(threads), 0, s, (const float*)a, (__nv_bfloat16*)y, (float*)state,
                  (const int32_t*)req_meta, (const int32_t*)slots, (const int32_t*)positions, (const float*)bias, W);
    else
        MM_REQUIRE(false, "mingru: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

MM_EXPORT int mm_mingru_chunked(const void* a, void* y, int dtype, void* state, void* A, void* B, const void* chunk_meta,
                                const void* req_chunks, const void* slots, const void* positions, const void* bias, int n_requests,
                                int n_chunks, int W, void* stream) {
    MM_REQUIRE(n_requests >= 0 && n_chunks >= 0 && W > 0, "mingru: bad sizes");
    if (n_requests == 0 || n_chunks == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = W >= 128 ? 128 : 64;
    const int bx = ceil_div(W, threads);
    if (dtype == MM_BF16)
        mm_launch(mingru_chunk_reduce_kernel<true>, dim3(bx, n_chunks), dim3(threads), 0, s, (const float*)a, (float*)A, (float*)B,
                  (const int32_t*)chunk_meta, (const float*)bias, W);
    else
        mm_launch(mingru_chunk_reduce_kernel<false>, dim3(bx, n_chunks), dim3(threads), 0, s, (const float*)a, (float*)A, (float*)B,
                  (const int32_t*)chunk_meta, (const float*)bias, W);
    MM_CHECK_LAUNCH();
    mm_launch(mingru_chunk_carry_kernel, dim3(bx, n_requests), dim3(threads), 0, s, (const float*)A, (float*)B, (float*)state,
              (const int32_t*)req_chunks, (const int32_t*)chunk_meta, (const int32_t*)slots, (const int32_t*)positions, W);
    MM_CHECK_LAUNCH();
    if (dtype == MM_F32)
        mm_launch(mingru_chunk_apply_kernel<float>, dim3(bx, n_chunks), dim3(threads), 0, s, (const float*)a, (const float*)B,
                  (float*)y, (const int32_t*)chunk_meta, (const float*)bias, W);
    else if (dtype == MM_BF16)
        mm_launch(mingru_chunk_apply_kernel<__nv_bfloat16>, dim3(bx, n_chunks), dim3(threads), 0, s, (const float*)a,
                  (const float*)B, (__nv_bfloat16*)y, (const int32_t*)chunk_meta, (const float*)bias, W);
    else
        MM_REQUIRE(false, "mingru: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}
