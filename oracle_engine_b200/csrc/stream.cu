// Row-wise kernels on the float32 residual stream for layers that norm in groups, average over depth, take a
// per-token side input and use a polynomial activation with norms.
//
//   group_rmsnorm       (x's row stride free) y = G(x; w): the row cut into `groups` equal consecutive parts, each part divided by its own
//                       sqrt(mean(part^2) + eps), the whole times w; x float32, y float32 or bfloat16
//   group_rmsnorm_add   dst (+)= coef * G(y; w), all float32; optionally also leaves the new dst rounded to bfloat16
//   poly_norm           out = a R(z) + b R(z^2) + c R(z^3) + e per row, R(u) = u / sqrt(mean(u^2) + eps), powers element
//                       by element; z float32, the four numbers read from device memory
//   side_gate           g[t, j] = gelu_tanh(u[t, j]) * table[token[t], off + j]
//   depth_average       hist[n] = x;  x = sum_{j <= n} w[j] hist[j]   (terms added in order of j)
//
// Every sum over a row is taken in an order fixed by the row's size alone, so a row's result does not depend on
// the other rows of the step.
#include "common.cuh"

namespace {

// One block per row; warp g takes the parts g, g + warps, ... : a part's sum is one warp's sum.  VEC: the part's size is
// a multiple of 4 and every row starts on a 16-byte boundary, so a lane moves 4 values at a time (a lane's sum then runs
// over the values 4 lane + {0..3}, 4 (lane + 32) + {0..3}, ...: another fixed order, chosen by the sizes alone).
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
group_rmsnorm_kernel(T* y, const float* x, long long ldx, const float* __restrict__ w, int D, int groups, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int gs = D / groups;
    const float* xr = x + (size_t)blockIdx.x * ldx;
    T* yr = y + (size_t)blockIdx.x * D;
    for (int g = warp; g < groups; g += nw) {
        const float* xp = xr + (size_t)g * gs;
        float ss = 0.f;
        if (VEC) {
            const float4* xp4 = reinterpret_cast<const float4*>(xp);
            const float4* w4 = reinterpret_cast<const float4*>(w + (size_t)g * gs);
            for (int d = lane; d < gs / 4; d += 32) {
                const float4 v = xp4[d];
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
            ss = warp_sum(ss);
            const float s = 1.f / sqrtf(ss / (float)gs + eps);
            for (int d = lane; d < gs / 4; d += 32) {
                const float4 v = xp4[d], ww = w4[d];
                store4(yr + (size_t)g * gs + 4 * d, (v.x * s) * ww.x, (v.y * s) * ww.y, (v.z * s) * ww.z, (v.w * s) * ww.w);
            }
            continue;
        }
        for (int d = lane; d < gs; d += 32) { const float v = xp[d]; ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        const float s = 1.f / sqrtf(ss / (float)gs + eps);
        for (int d = lane; d < gs; d += 32) yr[(size_t)g * gs + d] = from_f32<T>((xp[d] * s) * w[(size_t)g * gs + d]);
    }
}

template <bool VEC>
__global__ void __launch_bounds__(256)
group_rmsnorm_add_kernel(float* dst, const float* y, const float* __restrict__ w, int D, int groups, float eps,
                         float coef, int accumulate, bf16* cast) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int gs = D / groups;
    const float* yr = y + (size_t)blockIdx.x * D;
    float* dr = dst + (size_t)blockIdx.x * D;
    for (int g = warp; g < groups; g += nw) {
        const float* yp = yr + (size_t)g * gs;
        float ss = 0.f;
        if (VEC) {
            const float4* yp4 = reinterpret_cast<const float4*>(yp);
            const float4* w4 = reinterpret_cast<const float4*>(w + (size_t)g * gs);
            for (int d = lane; d < gs / 4; d += 32) {
                const float4 v = yp4[d];
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
            ss = warp_sum(ss);
            const float s = 1.f / sqrtf(ss / (float)gs + eps);
            for (int d = lane; d < gs / 4; d += 32) {
                const size_t at = (size_t)g * gs + 4 * d;
                const float4 v = yp4[d], ww = w4[d];
                float4 r = make_float4(coef * ((v.x * s) * ww.x), coef * ((v.y * s) * ww.y), coef * ((v.z * s) * ww.z),
                                       coef * ((v.w * s) * ww.w));
                if (accumulate) {
                    const float4 old = *reinterpret_cast<const float4*>(dr + at);
                    r.x = old.x + r.x; r.y = old.y + r.y; r.z = old.z + r.z; r.w = old.w + r.w;
                }
                *reinterpret_cast<float4*>(dr + at) = r;
                if (cast) store4(cast + (size_t)blockIdx.x * D + at, r.x, r.y, r.z, r.w);
            }
            continue;
        }
        for (int d = lane; d < gs; d += 32) { const float v = yp[d]; ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        const float s = 1.f / sqrtf(ss / (float)gs + eps);
        for (int d = lane; d < gs; d += 32) {
            const size_t at = (size_t)g * gs + d;
            const float add = coef * ((yp[d] * s) * w[at]);
            const float v = accumulate ? dr[at] + add : add;
            dr[at] = v;
            if (cast) cast[(size_t)blockIdx.x * D + at] = __float2bfloat16_rn(v);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
poly_norm_kernel(T* out, const float* z, long long ldz, const float* __restrict__ coef, int F, float eps) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* zr = z + (size_t)blockIdx.x * ldz;
    T* o = out + (size_t)blockIdx.x * F;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int d = threadIdx.x; d < F; d += blockDim.x) {
        const float v = zr[d], v2 = v * v, v3 = v2 * v;
        s2 += v2;
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v3, v3, s6);
    }
    s2 = block_sum(s2, red);
    s4 = block_sum(s4, red);
    s6 = block_sum(s6, red);
    const float r1 = coef[0] / sqrtf(s2 / (float)F + eps), r2 = coef[1] / sqrtf(s4 / (float)F + eps),
                r3 = coef[2] / sqrtf(s6 / (float)F + eps), e = coef[3];
    for (int d = threadIdx.x; d < F; d += blockDim.x) {
        const float v = zr[d], v2 = v * v;
        o[d] = from_f32<T>(((v * r1 + v2 * r2) + (v2 * v) * r3) + e);
    }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(256)
side_gate_kernel(T* g, const float* u, const T* __restrict__ table, long long ld_table, int off, int dim,
                 const int* __restrict__ token, const int* __restrict__ tok_seq, int vocab, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)n_tokens * dim;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / dim;
        const int j = (int)(e % dim);
        const int id = token[t];
        float v = 0.f;
        if (tok_seq[t] >= 0 && id >= 0 && id < vocab)
            v = gelu_tanh_f(u[e]) * to_f32(table[(size_t)id * ld_table + off + j]);
        g[e] = from_f32<T>(v);
    }
}

__global__ void __launch_bounds__(256)
depth_average_kernel(float* x, float* hist, long long layer_stride, const float* __restrict__ w, int n, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const float cur = x[e];
        hist[(size_t)n * layer_stride + e] = cur;
        float acc = 0.f;
        for (int j = 0; j < n; j++) acc = fmaf(w[j], hist[(size_t)j * layer_stride + e], acc);
        x[e] = fmaf(w[n], cur, acc);
    }
}

unsigned blocks_for(size_t total) {
    size_t b = (total + 255) / 256;
    if (b > 148 * 16) b = 148 * 16;
    return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace

extern "C" {

// whether every row of a [rows, D] tensor with row stride ld (values) and every part of it starts on a 16-byte boundary
static bool rows_of_4(const void* p, long long ld, int D, int groups) {
    return (D / groups) % 4 == 0 && ld % 4 == 0 && (uintptr_t)p % 16 == 0;
}

int oe_group_rmsnorm_f32(float* y, const float* x, long long ldx, const float* w, int rows, int D, int groups, float eps, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (groups < 1 || D < 1 || D % groups) return OE_ERR_UNSUPPORTED;
    if (rows_of_4(x, ldx, D, groups) && rows_of_4(y, D, D, groups) && rows_of_4(w, D, D, groups))
        return oe_launch(group_rmsnorm_kernel<float, true>, dim3(rows), dim3(groups >= 8 ? 256 : 128), 0, st, y, x, ldx, w, D, groups, eps);
    return oe_launch(group_rmsnorm_kernel<float, false>, dim3(rows), dim3(groups >= 8 ? 256 : 128), 0, st, y, x, ldx, w, D, groups, eps);
}
int oe_group_rmsnorm_bf16(bf16* y, const float* x, long long ldx, const float* w, int rows, int D, int groups, float eps, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (groups < 1 || D < 1 || D % groups) return OE_ERR_UNSUPPORTED;
    if (rows_of_4(x, ldx, D, groups) && (uintptr_t)y % 8 == 0 && rows_of_4(w, D, D, groups))
        return oe_launch(group_rmsnorm_kernel<bf16, true>, dim3(rows), dim3(groups >= 8 ? 256 : 128), 0, st, y, x, ldx, w, D, groups, eps);
    return oe_launch(group_rmsnorm_kernel<bf16, false>, dim3(rows), dim3(groups >= 8 ? 256 : 128), 0, st, y, x, ldx, w, D, groups, eps);
}
int oe_group_rmsnorm_add(float* dst, const float* y, const float* w, int rows, int D, int groups, float eps, float coef,
                         int accumulate, bf16* cast, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (groups < 1 || D < 1 || D % groups) return OE_ERR_UNSUPPORTED;
    if (rows_of_4(dst, D, D, groups) && rows_of_4(y, D, D, groups) && rows_of_4(w, D, D, groups) && (uintptr_t)cast % 8 == 0)
        return oe_launch(group_rmsnorm_add_kernel<true>, dim3(rows), dim3(groups >= 8 ? 256 : 128), 0, st, dst, y, w, D, groups, eps,
                         coef, accumulate, cast);
    return oe_launch(group_rmsnorm_add_kernel<false>, dim3(rows), dim3(groups >= 8 ? 256 : 128), 0, st, dst, y, w, D, groups, eps, coef,
                     accumulate, cast);
}
int oe_poly_norm_f32(float* out, const float* z, long long ldz, const float* coef, int rows, int F, float eps, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (F < 1) return OE_ERR_UNSUPPORTED;
    return oe_launch(poly_norm_kernel<float>, dim3(rows), dim3(256), 0, st, out, z, ldz, coef, F, eps);
}
int oe_poly_norm_bf16(bf16* out, const float* z, long long ldz, const float* coef, int rows, int F, float eps, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (F < 1) return OE_ERR_UNSUPPORTED;
    return oe_launch(poly_norm_kernel<bf16>, dim3(rows), dim3(256), 0, st, out, z, ldz, coef, F, eps);
}
int oe_side_gate_f32(float* g, const float* u, const float* table, long long ld_table, int off, int dim, const int* token,
                     const int* tok_seq, int vocab, int n_tokens, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (dim < 1) return OE_ERR_UNSUPPORTED;
    return oe_launch(side_gate_kernel<float>, dim3(blocks_for((size_t)n_tokens * dim)), dim3(256), 0, st, g, u, table, ld_table,
                     off, dim, token, tok_seq, vocab, n_tokens);
}
int oe_side_gate_bf16(bf16* g, const float* u, const bf16* table, long long ld_table, int off, int dim, const int* token,
                      const int* tok_seq, int vocab, int n_tokens, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (dim < 1) return OE_ERR_UNSUPPORTED;
    return oe_launch(side_gate_kernel<bf16>, dim3(blocks_for((size_t)n_tokens * dim)), dim3(256), 0, st, g, u, table, ld_table,
                     off, dim, token, tok_seq, vocab, n_tokens);
}
int oe_depth_average(float* x, float* hist, long long layer_stride, const float* w, int n, long long total, cudaStream_t st) {
    if (total <= 0) return 0;
    if (n < 0) return OE_ERR_UNSUPPORTED;
    return oe_launch(depth_average_kernel, dim3(blocks_for((size_t)total)), dim3(256), 0, st, x, hist, layer_stride, w, n,
                     (size_t)total);
}

}  // extern "C"
