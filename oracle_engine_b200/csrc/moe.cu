// Routing of a mixture of experts, and the activation of its experts computed side by side.
//
//   moe_route       one warp per token.  z [T, ldz] float32 holds the router's logits of E experts (and, when
//                   has_gate, one more column: the logit of the shared expert's gate).  The `top` largest logits
//                   choose the experts (of equal logits the lower index first); their weights are the softmax
//                   over the chosen logits alone.  Written: idx [T, top] and wt [T, top] (either may be null), and
//                   dense [T, E + (has_gate != 0)]: an expert's weight where it was chosen, zero elsewhere, and
//                   in the last column sigmoid(gate logit) (has_gate 1) or one (has_gate 2: a shared expert without
//                   a gate; z then holds no column for it).  mode 1: the weight of a chosen expert is the sigmoid
//                   of its own logit, not renormalised (the choice is by the same order).  With `bias` (one float32
//                   per expert, mode 1 only) the choice is by sigmoid(z) + bias and the weight stays sigmoid(z).
//   moe_dense_act   gu [T, 2 F] holds, for F = E ff + shared_ff columns, the gate rows and, F columns further, the
//                   up rows of all experts (expert e owns columns e ff .. (e + 1) ff - 1, the shared expert the last
//                   shared_ff).  a[t, c] = silu(gate) * up * dense[t, expert of c]: the experts a token did not
//                   choose contribute zeros to the one product with all down matrices that follows.  scale_input:
//                   the weight multiplies the expert's input instead of its output, a = silu(w gate) * (w up).
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* z, long long ldz, int E, int top, int has_gate, int mode, int* idx, float* wt, float* dense,
                 const int* __restrict__ tok_seq, int n_tokens, const float* __restrict__ bias) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= n_tokens) return;
    const int W = E + (has_gate ? 1 : 0);
    float* drow = dense + (size_t)t * W;
    for (int e = lane; e < W; e += 32) drow[e] = 0.f;
    if (tok_seq[t] < 0) {
        for (int j = lane; j < top; j += 32) {
            if (idx) idx[(size_t)t * top + j] = 0;
            if (wt) wt[(size_t)t * top + j] = 0.f;
        }
        return;
    }
    __syncwarp();
    const float* zr = z + (size_t)t * ldz;
    unsigned taken = 0;                      // bit i: this lane's element lane + 32 i is chosen already
    float zmax = 0.f, sum = 0.f;
    // pass 1: choose; the first chosen logit is the largest and anchors the exponentials
    for (int j = 0; j < top; j++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = 0, e = lane; e < E; e += 32, i++) {
            if (taken >> i & 1u) continue;
            const float v = bias ? 1.f / (1.f + expf(-zr[e])) + bias[e] : zr[e];
            if (v > best || (v == best && e < bi)) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) break;         // fewer experts than `top`
        if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
        if (j == 0) zmax = best;
        const float p = mode == 1 ? 1.f / (1.f + expf(-(bias ? zr[bi] : best))) : expf(best - zmax);
        sum += p;
        if (lane == 0) {
            if (idx) idx[(size_t)t * top + j] = bi;
            drow[bi] = p;
            if (wt) wt[(size_t)t * top + j] = p;
        }
    }
    __syncwarp();
    const float inv = mode == 1 ? 1.f : 1.f / sum;
    for (int i = 0, e = lane; e < E; e += 32, i++)
        if (taken >> i & 1u) drow[e] *= inv;
    if (wt) for (int j = lane; j < top; j += 32) wt[(size_t)t * top + j] *= inv;
    if (has_gate && lane == 0) drow[E] = has_gate == 2 ? 1.f : 1.f / (1.f + expf(-zr[E]));
}

// One thread takes 8 consecutive columns of one token (16 bytes of bfloat16) where an expert's columns come in
// multiples of 8, else one column; the columns of an expert the token did not choose are written as zeros without
// their gate and up values being read.
template <typename T, int V>
__global__ void __launch_bounds__(256)
moe_dense_act_kernel(T* a, const T* gu, const float* dense, int n_tokens, int F, int E, int ff, int W, int scale_input,
                     int act, float limit) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = F / V;
    const size_t total = (size_t)n_tokens * per_row;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / per_row;
        const int c = (int)(e % per_row) * V;
        int grp = c / ff;
        if (grp > E) grp = E;
        const float w = grp < W ? dense[t * W + grp] : 0.f;
        T out[V];
        if (w != 0.f) {
            T g[V], u[V];
            if (V == 8) {
                *reinterpret_cast<uint4*>(g) = *reinterpret_cast<const uint4*>(gu + t * 2 * F + c);
                *reinterpret_cast<uint4*>(u) = *reinterpret_cast<const uint4*>(gu + t * 2 * F + F + c);
            } else {
                g[0] = gu[t * 2 * F + c];
                u[0] = gu[t * 2 * F + F + c];
            }
#pragma unroll
            for (int i = 0; i < V; i++) {
                if (act == 1) {
                    const float gf = fminf(to_f32(g[i]), limit);
                    const float uf = fminf(fmaxf(to_f32(u[i]), -limit), limit);
                    out[i] = from_f32<T>(gf / (1.f + expf(-1.702f * gf)) * (uf + 1.f) * w);
                } else if (scale_input) {
                    const float gf = to_f32(g[i]) * w;
                    out[i] = from_f32<T>(gf / (1.f + expf(-gf)) * (to_f32(u[i]) * w));
                } else {
                    const float gf = to_f32(g[i]);
                    out[i] = from_f32<T>(gf / (1.f + expf(-gf)) * to_f32(u[i]) * w);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < V; i++) out[i] = from_f32<T>(0.f);
        }
        if (V == 8) *reinterpret_cast<uint4*>(a + t * F + c) = *reinterpret_cast<uint4*>(out);
        else a[t * F + c] = out[0];
    }
}

template <typename T>
int launch_act(T* a, const T* gu, const float* dense, int n_tokens, int F, int E, int ff, int W, int scale_input,
               int act, float limit, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (F < 1 || ff < 1 || E < 0 || act < 0 || act > 1 || (act == 1 && scale_input)) return OE_ERR_UNSUPPORTED;
    // 16-byte pieces: bfloat16, every expert's columns and the row a multiple of 8, aligned pointers
    const bool vec = sizeof(T) == 2 && ff % 8 == 0 && F % 8 == 0 && !(((uintptr_t)a | (uintptr_t)gu) & 15);
    const size_t total = (size_t)n_tokens * (vec ? F / 8 : F);
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (vec)
        return oe_launch(moe_dense_act_kernel<T, 8>, dim3((unsigned)blocks), dim3(256), 0, st, a, gu, dense, n_tokens, F, E, ff, W, scale_input, act, limit);
    return oe_launch(moe_dense_act_kernel<T, 1>, dim3((unsigned)blocks), dim3(256), 0, st, a, gu, dense, n_tokens, F, E, ff, W, scale_input, act, limit);
}

}  // namespace

extern "C" {

int oe_moe_route(const float* z, long long ldz, int E, int top, int has_gate, int mode, int* idx, float* wt, float* dense,
                 const int* tok_seq, int n_tokens, const float* bias, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (E < 1 || E > 1024 || top < 1 || (bias != nullptr && mode != 1)) return OE_ERR_UNSUPPORTED;
    return oe_launch(moe_route_kernel, dim3((n_tokens + 3) / 4), dim3(128), 0, st, z, ldz, E, top, has_gate, mode, idx, wt, dense,
                     tok_seq, n_tokens, bias);
}
int oe_moe_dense_act_f32(float* a, const float* gu, const float* dense, int n_tokens, int F, int E, int ff, int W,
                         int scale_input, int act, float limit, cudaStream_t st) {
    return launch_act<float>(a, gu, dense, n_tokens, F, E, ff, W, scale_input, act, limit, st);
}
int oe_moe_dense_act_bf16(bf16* a, const bf16* gu, const float* dense, int n_tokens, int F, int E, int ff, int W,
                          int scale_input, int act, float limit, cudaStream_t st) {
    return launch_act<bf16>(a, gu, dense, n_tokens, F, E, ff, W, scale_input, act, limit, st);
}

}  // extern "C"
