// Norms and gates that stand between a mixer's heads and its output projection, and the mean of normed branches.
//
// (1) gated group norm:  y[t, g, :] = x[t, g, :] / rms(x[t, g, :]) * w * act(gate[t, g, :])
//     over `groups` groups of `gs` numbers per row (a head each, or the whole row as one group); the division, the
//     weight and the gate are each optional; w is one vector of gs for all groups (w_stride 0) or one per group
//     (w_stride gs); act is silu or the logistic function.  Arithmetic in fp32, output in the activation dtype.
// (2) mean of normed rows:  y[t, :] = scale * (a[t, :] / rms(a[t, :]) * wa + b[t, :] / rms(b[t, :]) * wb).
#include "common.cuh"

__device__ __forceinline__ float ng_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename TI, typename TG, typename TO>
__global__ void gated_group_norm_kernel(const TI* __restrict__ x, int ldx, const TG* __restrict__ gate, int ldg, const float* __restrict__ w,
                                        int w_stride, TO* __restrict__ out, int gs, float eps, int normalize, int act) {
    __shared__ float scratch[32];
    const int g = blockIdx.y;
    const size_t t = blockIdx.x;
    const TI* xr = x + t * ldx + (size_t)g * gs;
    float inv = 1.0f;
    if (normalize) {
        float ss = 0.0f;
        for (int d = threadIdx.x; d < gs; d += blockDim.x) {
            const float a = to_f32<TI>(xr[d]);
            ss = fmaf(a, a, ss);
        }
        ss = block_sum(ss, scratch);
        inv = 1.0f / sqrtf(ss / (float)gs + eps);
    }
    const TG* gr = gate ? gate + t * ldg + (size_t)g * gs : nullptr;
    const float* wr = w ? w + (size_t)g * w_stride : nullptr;
    TO* o = out + (t * gridDim.y + g) * gs;
    for (int d = threadIdx.x; d < gs; d += blockDim.x) {
        float y = to_f32<TI>(xr[d]) * inv;
        if (wr) y *= wr[d];
        if (gr) {
            const float z = to_f32<TG>(gr[d]);
            y *= act == 1 ? z * ng_sigmoid(z) : ng_sigmoid(z);
        }
        o[d] = from_f32<TO>(y);
    }
}

template <typename TI, typename TG, typename TO>
static void ggn_launch(dim3 grid, int threads, cudaStream_t s, const void* x, int ldx, const void* gate, int ldg, const void* w, int w_stride,
                       void* out, int gs, float eps, int normalize, int act) {
    mm_launch(gated_group_norm_kernel<TI, TG, TO>, grid, dim3(threads), 0, s, (const TI*)x, ldx, (const TG*)gate, ldg, (const float*)w, w_stride,
              (TO*)out, gs, eps, normalize, act);
}

// x [n, ldx] of x_dtype, gate [n, ldg] of gate_dtype or null, w fp32 or null, out [n, groups * gs] of out_dtype
MM_EXPORT int mm_gated_group_norm(const void* x, int x_dtype, int ldx, const void* gate, int gate_dtype, int ldg, const void* w, int w_stride,
                                  void* out, int out_dtype, int n, int groups, int gs, float eps, int normalize, int act, void* stream) {
    MM_REQUIRE(n >= 0 && groups > 0 && gs > 0 && ldx >= groups * gs, "gated norm: bad sizes");
    MM_REQUIRE(gate == nullptr || (ldg >= groups * gs && (act == 1 || act == 2)), "gated norm: the gate's activation is 1 (silu) or 2 (logistic)");
    MM_REQUIRE(w_stride == 0 || w_stride == gs, "gated norm: one weight vector for all groups or one per group");
    if (n == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n, groups);
    const int threads = gs >= 1024 ? 256 : (gs >= 128 ? 128 : (gs > 32 ? 64 : 32));
    const int gd = gate ? gate_dtype : MM_F32;
#define GGN(TI, TG, TO) ggn_launch<TI, TG, TO>(grid, threads, s, x, ldx, gate, ldg, w, w_stride, out, gs, eps, normalize, act)
    typedef __nv_bfloat16 bf;
    if (x_dtype == MM_F32 && gd == MM_F32 && out_dtype == MM_F32) GGN(float, float, float);
    else if (x_dtype == MM_F32 && gd == MM_F32 && out_dtype == MM_BF16) GGN(float, float, bf);
    else if (x_dtype == MM_F32 && gd == MM_BF16 && out_dtype == MM_BF16) GGN(float, bf, bf);
    else if (x_dtype == MM_BF16 && gd == MM_F32 && out_dtype == MM_BF16) GGN(bf, float, bf);
    else if (x_dtype == MM_BF16 && gd == MM_BF16 && out_dtype == MM_BF16) GGN(bf, bf, bf);
    else MM_REQUIRE(false, "gated norm: this combination of dtypes is not built");
#undef GGN
    MM_CHECK_LAUNCH();
    return MM_OK;
}

template <typename T>
__global__ void normed_mean2_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ wa, const float* __restrict__ wb,
                                    T* __restrict__ out, int d, float eps, float scale) {
    __shared__ float scratch[32];
    const size_t t = blockIdx.x;
    const T* ar = a + t * d;
    const T* br = b + t * d;
    float sa = 0.0f, sb = 0.0f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float x = to_f32<T>(ar[i]), y = to_f32<T>(br[i]);
        sa = fmaf(x, x, sa);
        sb = fmaf(y, y, sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ia = 1.0f / sqrtf(sa / (float)d + eps), ib = 1.0f / sqrtf(sb / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        out[t * d + i] = from_f32<T>(scale * (to_f32<T>(ar[i]) * ia * wa[i] + to_f32<T>(br[i]) * ib * wb[i]));
}

MM_EXPORT int mm_normed_mean2(const void* a, const void* b, const void* wa, const void* wb, void* out, int dtype, int n, int d, float eps,
                              float scale, void* stream) {
    MM_REQUIRE(n >= 0 && d > 0, "normed mean: bad sizes");
    if (n == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 2048 ? 256 : 128;
    if (dtype == MM_F32)
        mm_launch(normed_mean2_kernel<float>, dim3(n), dim3(threads), 0, s, (const float*)a, (const float*)b, (const float*)wa, (const float*)wb,
                  (float*)out, d, eps, scale);
    else if (dtype == MM_BF16)
        mm_launch(normed_mean2_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, s, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                  (const float*)wa, (const float*)wb, (__nv_bfloat16*)out, d, eps, scale);
    else
        MM_REQUIRE(false, "normed mean: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}
