// Bias and activation of a feed-forward's hidden rows: out = act(x + bias), fp32 arithmetic, rounded once.
//
//   relu2      max(z, 0)^2
//   gelu_tanh  0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
//   silu       z / (1 + exp(-z))
//   relu       max(z, 0)
#include "common.cuh"

#define ACT_RELU2 0
#define ACT_GELU_TANH 1
#define ACT_SILU 2
#define ACT_RELU 3

__device__ __forceinline__ float apply_act(float z, int act) {
    switch (act) {
        case ACT_RELU2: { const float r = fmaxf(z, 0.0f); return r * r; }
        case ACT_GELU_TANH: return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        case ACT_SILU: return z / (1.0f + expf(-z));
        default: return fmaxf(z, 0.0f);
    }
}

template <typename T, typename BT>
__global__ void bias_act_kernel(const T* __restrict__ x, const BT* __restrict__ bias, T* __restrict__ out, long long total,
                                int f, int act) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        float z = to_f32<T>(x[i]);
        if (bias != nullptr) z += to_f32<BT>(bias[i % f]);
        out[i] = from_f32<T>(apply_act(z, act));
    }
}

// bfloat16 rows whose width is a multiple of 8: 16-byte loads and stores
template <typename BT>
__global__ void bias_act_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, const BT* __restrict__ bias,
                                       __nv_bfloat16* __restrict__ out, long long total8, int f, int act) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += stride) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + i * 8);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const int col = (int)((i * 8) % f);
        uint4 res;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 z = __bfloat1622float2(p2[k]);
            if (bias != nullptr) {
                z.x += to_f32<BT>(bias[col + 2 * k]);
                z.y += to_f32<BT>(bias[col + 2 * k + 1]);
            }
            o2[k] = __floats2bfloat162_rn(apply_act(z.x, act), apply_act(z.y, act));
        }
        *reinterpret_cast<uint4*>(out + i * 8) = res;
    }
}

MM_EXPORT int mm_bias_act(const void* x, const void* bias, int bias_dtype, void* out, int dtype, int n, int f, int act, void* stream) {
    MM_REQUIRE(n >= 0 && f > 0 && act >= 0 && act <= 3, "bias_act: bad sizes or activation");
    if (n == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)n * f;
    const int threads = 256;
    if (dtype == MM_BF16 && f % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const long long total8 = total / 8;
        const int blocks = (int)min((long long)148 * 16, (total8 + threads - 1) / threads);
        if (bias_dtype == MM_BF16)
            mm_launch(bias_act_bf16x8_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)x,
                      (const __nv_bfloat16*)bias, (__nv_bfloat16*)out, total8, f, act);
        else
            mm_launch(bias_act_bf16x8_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)x, (const float*)bias,
                      (__nv_bfloat16*)out, total8, f, act);
        MM_CHECK_LAUNCH();
        return MM_OK;
    }
    const int blocks = (int)min((long long)148 * 16, (total + threads - 1) / threads);
    if (dtype == MM_F32 && bias_dtype == MM_F32)
        mm_launch(bias_act_kernel<float, float>, dim3(blocks), dim3(threads), 0, s, (const float*)x, (const float*)bias, (float*)out, total, f, act);
    else if (dtype == MM_BF16 && bias_dtype == MM_BF16)
        mm_launch(bias_act_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)x,
                  (const __nv_bfloat16*)bias, (__nv_bfloat16*)out, total, f, act);
    else if (dtype == MM_BF16 && bias_dtype == MM_F32)
        mm_launch(bias_act_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)x, (const float*)bias,
                  (__nv_bfloat16*)out, total, f, act);
    else
        MM_REQUIRE(false, "bias_act: unsupported dtype combination");
    MM_CHECK_LAUNCH();
    return MM_OK;
}
