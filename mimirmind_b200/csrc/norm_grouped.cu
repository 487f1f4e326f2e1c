// RMS norm in groups, and the chain "norm a branch, add it to the residual stream, norm the sum".
//
// A row of width d is cut into `groups` equal consecutive parts; each part is divided by its own
// sqrt(mean(part^2) + eps) and the whole row is multiplied by a weight.  One block per row.  In one launch:
//
//   if branch:  residual += w_post ? gnorm(branch) * w_post : branch        (fp32, in place)
//   if w_next:  out = gnorm(residual) * w_next                              (activation dtype)
//
// so a layer that norms a sublayer's output before the residual add and norms again before the next sublayer makes
// one trip over the row.  With `rows`, output row i is made from source row rows[i] and nothing is added.
// All arithmetic is fp32; sums run in a fixed order that depends on the width, the groups and the block only.
#include "common.cuh"

#define GN_MAX_WARPS 16

// Sum of squares of every group of the cached row -> inv[g] = 1 / sqrt(mean + eps).  The warps of the block are
// shared out over the groups (S warps per group when there are at least as many warps as groups, else every warp
// takes whole groups in turn); partial sums are added in segment order.
__device__ __forceinline__ void group_inverse_rms(const float* __restrict__ row, int d, int groups, float eps,
                                                  float* __restrict__ part, float* __restrict__ inv) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int gs = d / groups;
    if (groups <= nwarps) {
        const int S = nwarps / groups;
        const int seg = (gs + S - 1) / S;
        if (warp < groups * S) {
            const int g = warp / S, s = warp - g * S;
            const int lo = g * gs + s * seg, hi = min(g * gs + gs, lo + seg);
            float ss = 0.0f;
            for (int k = lo + lane; k < hi; k += 32) ss = fmaf(row[k], row[k], ss);
            ss = warp_sum(ss);
            if (lane == 0) part[warp] = ss;
        }
        __syncthreads();
        if (threadIdx.x < groups) {
            float t = 0.0f;
            for (int s = 0; s < S; ++s) t += part[threadIdx.x * S + s];
            inv[threadIdx.x] = 1.0f / sqrtf(t / (float)gs + eps);
        }
    } else {
        for (int g = warp; g < groups; g += nwarps) {
            float ss = 0.0f;
            for (int k = g * gs + lane; k < g * gs + gs; k += 32) ss = fmaf(row[k], row[k], ss);
            ss = warp_sum(ss);
            if (lane == 0) inv[g] = 1.0f / sqrtf(ss / (float)gs + eps);
        }
    }
    __syncthreads();
}

template <typename T, typename WT>
__global__ void group_norm_chain_kernel(float* __restrict__ residual, const T* __restrict__ branch,
                                        const WT* __restrict__ w_post, const WT* __restrict__ w_next,
                                        const int32_t* __restrict__ rows, T* __restrict__ out, int d, int groups, float eps) {
    extern __shared__ float gn_smem[];      // row [d], inv [groups], part [GN_MAX_WARPS]
    float* row = gn_smem;
    float* inv = gn_smem + d;
    float* part = inv + groups;
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    float* res = residual + r * d;
    const int gs = d / groups;
    if (branch != nullptr) {
        const T* b = branch + r * d;
        for (int k = threadIdx.x; k < d; k += blockDim.x) row[k] = to_f32<T>(b[k]);
        __syncthreads();
        if (w_post != nullptr) {
            group_inverse_rms(row, d, groups, eps, part, inv);
            for (int k = threadIdx.x; k < d; k += blockDim.x) {
                const float v = res[k] + row[k] * inv[k / gs] * to_f32<WT>(w_post[k]);
                res[k] = v;
                row[k] = v;
            }
        } else {
            for (int k = threadIdx.x; k < d; k += blockDim.x) {
                const float v = res[k] + row[k];
                res[k] = v;
                row[k] = v;
            }
        }
    } else {
        for (int k = threadIdx.x; k < d; k += blockDim.x) row[k] = res[k];
    }
    if (w_next == nullptr) return;
    __syncthreads();
    group_inverse_rms(row, d, groups, eps, part, inv);
    T* o = out + (size_t)i * d;
    for (int k = threadIdx.x; k < d; k += blockDim.x) o[k] = from_f32<T>(row[k] * inv[k / gs] * to_f32<WT>(w_next[k]));
}

// Plain grouped norm of rows in the activation dtype (no residual): out = gnorm(x) * w.
template <typename T, typename WT>
__global__ void group_norm_rows_kernel(const T* __restrict__ x, const WT* __restrict__ w, T* __restrict__ out, int d,
                                       int groups, float eps) {
    extern __shared__ float gn_smem[];
    float* row = gn_smem;
    float* inv = gn_smem + d;
    float* part = inv + groups;
    const size_t i = blockIdx.x;
    const int gs = d / groups;
    for (int k = threadIdx.x; k < d; k += blockDim.x) row[k] = to_f32<T>(x[i * d + k]);
    __syncthreads();
    group_inverse_rms(row, d, groups, eps, part, inv);
    for (int k = threadIdx.x; k < d; k += blockDim.x) out[i * d + k] = from_f32<T>(row[k] * inv[k / gs] * to_f32<WT>(w[k]));
}

// bfloat16 activations, width a multiple of 256 per group and at most 8192: a thread keeps 8 consecutive elements of the
// row in registers (16-byte loads and stores), a warp's 256 elements lie in one group, and a group's sum is the sum of
// its warps' partial sums in warp order.  One trip over the row for both norms.
template <typename WT>
__device__ __forceinline__ void load_weight8(const WT* __restrict__ w, float* f);
template <>
__device__ __forceinline__ void load_weight8<float>(const float* __restrict__ w, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(w), b = *reinterpret_cast<const float4*>(w + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load_weight8<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, float* f) {
    const uint4 raw = *reinterpret_cast<const uint4*>(w);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 x = __bfloat1622float2(p2[k]);
        f[2 * k] = x.x;
        f[2 * k + 1] = x.y;
    }
}

__device__ __forceinline__ float group_inv_rms8(const float* v, int warps_per_group, int gs, float eps, float* part) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss = fmaf(v[k], v[k], ss);
    ss = warp_sum(ss);
    __syncthreads();                      // part may still be read from an earlier call
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    const int first = (warp / warps_per_group) * warps_per_group;
    float t = 0.0f;
    for (int w = 0; w < warps_per_group; ++w) t += part[first + w];
    return 1.0f / sqrtf(t / (float)gs + eps);
}

template <typename WT>
__global__ void group_norm_chain_bf16x8_kernel(float* __restrict__ residual, const __nv_bfloat16* __restrict__ branch,
                                               const WT* __restrict__ w_post, const WT* __restrict__ w_next,
                                               const int32_t* __restrict__ rows, __nv_bfloat16* __restrict__ out, int d,
                                               int groups, float eps) {
    __shared__ float part[32];
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    const int c = threadIdx.x * 8;
    const int gs = d / groups, wpg = gs / 256;
    float v[8], w[8];
    {
        const float4 a = *reinterpret_cast<const float4*>(residual + r * d + c);
        const float4 b = *reinterpret_cast<const float4*>(residual + r * d + c + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    if (branch != nullptr) {
        float bv[8];
        load_weight8<__nv_bfloat16>(branch + r * d + c, bv);
        if (w_post != nullptr) {
            const float inv = group_inv_rms8(bv, wpg, gs, eps, part);
            load_weight8<WT>(w_post + c, w);
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] += bv[k] * inv * w[k];
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] += bv[k];
        }
        *reinterpret_cast<float4*>(residual + r * d + c) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(residual + r * d + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    if (w_next == nullptr) return;
    const float inv = group_inv_rms8(v, wpg, gs, eps, part);
    load_weight8<WT>(w_next + c, w);
    uint4 res;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
    for (int k = 0; k < 4; ++k) o2[k] = __floats2bfloat162_rn(v[2 * k] * inv * w[2 * k], v[2 * k + 1] * inv * w[2 * k + 1]);
    *reinterpret_cast<uint4*>(out + (size_t)i * d + c) = res;
}

template <typename T, typename WT>
static int launch_chain(float* residual, const void* branch, const void* w_post, const void* w_next, const int32_t* rows,
                        void* out, int n, int d, int groups, float eps, cudaStream_t s) {
    const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
    const size_t smem = (size_t)(d + groups + GN_MAX_WARPS) * sizeof(float);
    auto kernel = group_norm_chain_kernel<T, WT>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            mm_set_last_error("group norm: the row does not fit into shared memory");
            return MM_ERR_UNSUPPORTED;
        }
    }
    mm_launch(kernel, dim3(n), dim3(threads), smem, s, residual, (const T*)branch, (const WT*)w_post, (const WT*)w_next, rows,
              (T*)out, d, groups, eps);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

MM_EXPORT int mm_group_norm_chain(void* residual, const void* branch, const void* w_post, const void* w_next, int weight_dtype,
                                  const void* rows, void* out, int dtype, int n_out, int d, int groups, float eps, void* stream) {
    MM_REQUIRE(n_out >= 0 && d > 0 && groups > 0 && d % groups == 0, "group norm: the width must be a multiple of the groups");
    MM_REQUIRE(branch == nullptr || rows == nullptr, "group norm: a gathered call adds nothing");
    MM_REQUIRE(w_next == nullptr || out != nullptr, "group norm: a norm needs an output");
    MM_REQUIRE(branch != nullptr || w_next != nullptr, "group norm: nothing to do");
    if (n_out == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    float* res = (float*)residual;
    const int32_t* rw = (const int32_t*)rows;
    if (dtype == MM_BF16 && (d / groups) % 256 == 0 && d <= 8192 &&
        (((uintptr_t)residual | (uintptr_t)branch | (uintptr_t)w_post | (uintptr_t)w_next | (uintptr_t)out) & 15) == 0) {
        if (weight_dtype == MM_BF16)
            mm_launch(group_norm_chain_bf16x8_kernel<__nv_bfloat16>, dim3(n_out), dim3(d / 8), 0, s, res, (const __nv_bfloat16*)branch,
                      (const __nv_bfloat16*)w_post, (const __nv_bfloat16*)w_next, rw, (__nv_bfloat16*)out, d, groups, eps);
        else
            mm_launch(group_norm_chain_bf16x8_kernel<float>, dim3(n_out), dim3(d / 8), 0, s, res, (const __nv_bfloat16*)branch,
                      (const float*)w_post, (const float*)w_next, rw, (__nv_bfloat16*)out, d, groups, eps);
        MM_CHECK_LAUNCH();
        return MM_OK;
    }
    if (dtype == MM_F32 && weight_dtype == MM_F32)
        return launch_chain<float, float>(res, branch, w_post, w_next, rw, out, n_out, d, groups, eps, s);
    if (dtype == MM_BF16 && weight_dtype == MM_BF16)
        return launch_chain<__nv_bfloat16, __nv_bfloat16>(res, branch, w_post, w_next, rw, out, n_out, d, groups, eps, s);
    if (dtype == MM_BF16 && weight_dtype == MM_F32)
        return launch_chain<__nv_bfloat16, float>(res, branch, w_post, w_next, rw, out, n_out, d, groups, eps, s);
    MM_REQUIRE(false, "group norm: unsupported dtype combination");
    return MM_OK;
}

MM_EXPORT int mm_group_norm_rows(const void* x, const void* w, int weight_dtype, void* out, int dtype, int n, int d, int groups,
                                 float eps, void* stream) {
    MM_REQUIRE(n >= 0 && d > 0 && groups > 0 && d % groups == 0, "group norm: the width must be a multiple of the groups");
    if (n == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
    const size_t smem = (size_t)(d + groups + GN_MAX_WARPS) * sizeof(float);
    MM_REQUIRE(smem <= 48 * 1024, "group norm: the row does not fit into shared memory");
    if (dtype == MM_F32 && weight_dtype == MM_F32)
        mm_launch(group_norm_rows_kernel<float, float>, dim3(n), dim3(threads), smem, s, (const float*)x, (const float*)w, (float*)out, d, groups, eps);
    else if (dtype == MM_BF16 && weight_dtype == MM_BF16)
        mm_launch(group_norm_rows_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(n), dim3(threads), smem, s, (const __nv_bfloat16*)x,
                  (const __nv_bfloat16*)w, (__nv_bfloat16*)out, d, groups, eps);
    else if (dtype == MM_BF16 && weight_dtype == MM_F32)
        mm_launch(group_norm_rows_kernel<__nv_bfloat16, float>, dim3(n), dim3(threads), smem, s, (const __nv_bfloat16*)x,
                  (const float*)w, (__nv_bfloat16*)out, d, groups, eps);
    else
        MM_REQUIRE(false, "group norm: unsupported dtype combination");
    MM_CHECK_LAUNCH();
    return MM_OK;
}
