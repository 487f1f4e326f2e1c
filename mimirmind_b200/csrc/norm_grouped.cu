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
