// Grouped-query attention whose keys and values have head sizes of their own (dk, dv) and lie in two tensors
// of the paged cache, with a partial rotation of q and k, a cap on the scores and a window.
//
//   rope_split_kv_write   rotates the first `rot` dimensions of every q and k head of the step's tokens
//                         (dimension i < rot/2 is paired with i + rot/2; the angle's cosine and sine come from
//                         a float32 table [positions, rot/2]); q is written back in place, k goes to the token's
//                         row of the key tensor [pages, G, PAGE, dk], v as projected to the value tensor
//                         [pages, G, PAGE, dv].
//   attn_split            one warp per (token, query head): s_j = scale q.k_j, then s_j <- cap tanh(s_j / cap)
//                         when cap > 0, for the keys pos - window < j <= pos (all keys up to pos when window
//                         is 0); online softmax in float32 over chunks of 32 keys at absolute multiples of 32,
//                         so a token's result does not depend on how the step was cut or batched.  The
//                         32-bit path's attention, and the bfloat16 path's for head sizes that the tensor-core
//                         kernel (attention_split_mma.cu) does not take.  `sinks` (null, or one float32 per query
//                         head): the softmax's denominator also holds exp(sinks[h]), a term without key or value.
//                         `unrot_cos`, `unrot_sin` (null, or float32 [positions, dv/2]): every head's result is turned
//                         back by its query's position, pair (m, m + dv/2), before it is stored.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

__device__ __forceinline__ long long split_row(const int* __restrict__ table_row, int pos, int g, int G, int d) {
    const int page = table_row[pos / OE_PAGE];
    if (page < 0) return -1;
    return (((long long)page * G + g) * OE_PAGE + (pos % OE_PAGE)) * d;
}

template <typename T>
__global__ void __launch_bounds__(128)
rope_split_kv_write_kernel(T* qkv, long long stride, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                           int rot, T* kcache, T* vcache, const int* __restrict__ tables, int max_pages,
                           const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, int H, int G, int dk,
                           int dv, int has_kv, int hpb) {
    // grid y: block y turns the heads y hpb .. (y + 1) hpb - 1 (q heads, then k heads); the last y copies v
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    if (b < 0) return;
    const int pos = tok_pos[t];
    T* row = qkv + (size_t)t * stride;
    const int half = rot / 2;
    const float* cr = cos_t + (size_t)pos * half;
    const float* sr = sin_t + (size_t)pos * half;
    const int* trow = tables + (size_t)b * max_pages;
    const int n_rot_heads = H + (has_kv ? G : 0);
    const int e_lo = blockIdx.y * hpb * dk;
    const int e_hi = min((int)(blockIdx.y + 1) * hpb, n_rot_heads) * dk;
    for (int e = e_lo + threadIdx.x; e < e_hi; e += blockDim.x) {
        const int hh = e / dk, i = e % dk;
        if (i >= half && i < rot) continue;                     // written by its partner
        T* src = row + (size_t)hh * dk;
        T* dst = src;
        if (hh >= H) {
            const long long off = split_row(trow, pos, hh - H, G, dk);
            if (off < 0) continue;
            dst = kcache + off;
        }
        if (i < half) {
            const float u = to_f32(src[i]), v = to_f32(src[i + half]);
            const float c = cr[i], s = sr[i];
            dst[i] = from_f32<T>(u * c - v * s);
            dst[i + half] = from_f32<T>(v * c + u * s);
        } else if (hh >= H) {
            dst[i] = src[i];
        }
    }
    if (has_kv && blockIdx.y == gridDim.y - 1) {
        const T* vsrc = row + (size_t)(H + G) * dk;
        for (int e = threadIdx.x; e < G * dv; e += blockDim.x) {
            const int g = e / dv, i = e % dv;
            const long long off = split_row(trow, pos, g, G, dv);
            if (off >= 0) vcache[off + i] = vsrc[e];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_split_kernel(T* out, const T* q, long long q_stride, const T* kcache, const T* vcache,
                  const int* __restrict__ tables, int max_pages, const int* __restrict__ tok_seq,
                  const int* __restrict__ tok_pos, int n_tokens, int H, int G, int dk, int dv, int window, float scale,
                  float cap, const float* __restrict__ sinks, const float* __restrict__ unrot_cos,
                  const float* __restrict__ unrot_sin) {
    extern __shared__ float qs_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    float* qs = qs_all + warp * max(dk, dv);
    T* o = out + (size_t)t * H * dv + (size_t)h * dv;
    const int b = tok_seq[t];
    if (b < 0) {
        for (int d = lane; d < dv; d += 32) o[d] = from_f32<T>(0.f);
        return;
    }
    const int pos = tok_pos[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int g = h / (H / G);
    const int* trow = tables + (size_t)b * max_pages;
    const T* qr = q + (size_t)t * q_stride + (size_t)h * dk;
    for (int d = lane; d < dk; d += 32) qs[d] = to_f32(qr[d]);
    __syncwarp();
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;

    // a sink: one more term exp(sinks[h]) in the denominator, with no key and no value
    float m = sinks ? sinks[h] : -INFINITY, l = sinks ? 1.f : 0.f;
    float acc[MAX_D / 32];
#pragma unroll
    for (int i = 0; i < MAX_D / 32; i++) acc[i] = 0.f;

    for (int c0 = (lo / 32) * 32; c0 <= pos; c0 += 32) {
        const int key = c0 + lane;
        float s = -INFINITY;
        if (key >= lo && key <= pos) {
            const long long off = split_row(trow, key, g, G, dk);
            if (off >= 0) {
                const T* kr = kcache + off;
                float dot = 0.f;
                for (int d = 0; d < dk; d++) dot = fmaf(qs[d], to_f32(kr[d]), dot);
                s = dot * scale;
                if (cap > 0.f) s = cap * tanhf(s * inv_cap);
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float alpha = expf(m - m_new);
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_D / 32; i++) acc[i] *= alpha;
        const int jmax = (pos - c0 < 31) ? pos - c0 : 31;
        for (int j = 0; j <= jmax; j++) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if (c0 + j < lo) continue;
            const long long voff = split_row(trow, c0 + j, g, G, dv);
            if (voff < 0) continue;
            const T* vr = vcache + voff;
#pragma unroll
            for (int i = 0; i < MAX_D / 32; i++) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = 1.f / l;
    if (unrot_cos != nullptr) {
        // the result turned back by the query's position: pair (m, m + dv/2) by minus the table's angle
        __syncwarp();
#pragma unroll
        for (int i = 0; i < MAX_D / 32; i++) {
            const int d = lane + 32 * i;
            if (d < dv) qs[d] = acc[i] * inv;
        }
        __syncwarp();
        const int half = dv / 2;
        const float* cr = unrot_cos + (size_t)pos * half;
        const float* sr = unrot_sin + (size_t)pos * half;
        for (int d = lane; d < dv; d += 32) {
            float r = qs[d];
            if (d < half) r = qs[d] * cr[d] + qs[d + half] * sr[d];
            else if (d < 2 * half) r = qs[d] * cr[d - half] - qs[d - half] * sr[d - half];
            o[d] = from_f32<T>(r);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < MAX_D / 32; i++) {
        const int d = lane + 32 * i;
        if (d < dv) o[d] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T>
int launch_rope(T* qkv, long long stride, const float* cos_t, const float* sin_t, int rot, T* kcache, T* vcache,
                const int* tables, int max_pages, const int* tok_seq, const int* tok_pos, int n_tokens, int H, int G,
                int dk, int dv, int has_kv, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (rot < 0 || rot % 2 || rot > dk || dk < 1 || dv < 1 || H < 1 || G < 1) return OE_ERR_UNSUPPORTED;
    // few tokens: a block per head, so that a token's loads are in flight together; many tokens: a block per token
    const int n_rot_heads = H + (has_kv ? G : 0);
    const int hpb = n_tokens <= 256 ? 1 : n_rot_heads;
    const int by = (n_rot_heads + hpb - 1) / hpb + (has_kv ? 1 : 0);
    if (by > 65535) return OE_ERR_UNSUPPORTED;
    return oe_launch(rope_split_kv_write_kernel<T>, dim3(n_tokens, by), dim3(128), 0, st, qkv, stride, cos_t, sin_t, rot,
                     kcache, vcache, tables, max_pages, tok_seq, tok_pos, H, G, dk, dv, has_kv, hpb);
}

template <typename T>
int launch_attn(T* out, const T* q, long long q_stride, const T* kcache, const T* vcache, const int* tables,
                int max_pages, const int* tok_seq, const int* tok_pos, int n_tokens, int H, int G, int dk, int dv,
                int window, float scale, float cap, const float* sinks, const float* unrot_cos, const float* unrot_sin,
                cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (unrot_cos == nullptr || unrot_sin == nullptr) unrot_cos = unrot_sin = nullptr;
    if (dk < 1 || dk > MAX_D || dv < 1 || dv > MAX_D || G < 1 || H % G) return OE_ERR_UNSUPPORTED;
    const long long items = (long long)n_tokens * H;
    const long long blocks = (items + WARPS - 1) / WARPS;
    if (blocks > 2147483647LL) return OE_ERR_UNSUPPORTED;
    return oe_launch(attn_split_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), WARPS * (dk > dv ? dk : dv) * sizeof(float), st, out, q,
                     q_stride, kcache, vcache, tables, max_pages, tok_seq, tok_pos, n_tokens, H, G, dk, dv, window, scale,
                     cap, sinks, unrot_cos, unrot_sin);
}

}  // namespace

extern "C" {
int oe_rope_split_kv_write_f32(float* qkv, long long stride, const float* cos_t, const float* sin_t, int rot,
                               float* kcache, float* vcache, const int* tables, int max_pages, const int* tok_seq,
                               const int* tok_pos, int n_tokens, int H, int G, int dk, int dv, int has_kv,
                               cudaStream_t st) {
    return launch_rope<float>(qkv, stride, cos_t, sin_t, rot, kcache, vcache, tables, max_pages, tok_seq, tok_pos,
                              n_tokens, H, G, dk, dv, has_kv, st);
}
int oe_rope_split_kv_write_bf16(bf16* qkv, long long stride, const float* cos_t, const float* sin_t, int rot,
                                bf16* kcache, bf16* vcache, const int* tables, int max_pages, const int* tok_seq,
                                const int* tok_pos, int n_tokens, int H, int G, int dk, int dv, int has_kv,
                                cudaStream_t st) {
    return launch_rope<bf16>(qkv, stride, cos_t, sin_t, rot, kcache, vcache, tables, max_pages, tok_seq, tok_pos,
                             n_tokens, H, G, dk, dv, has_kv, st);
}
int oe_attn_split_f32(float* out, const float* q, long long q_stride, const float* kcache, const float* vcache,
                      const int* tables, int max_pages, const int* tok_seq, const int* tok_pos, int n_tokens, int H,
                      int G, int dk, int dv, int window, float scale, float cap, const float* sinks,
                      const float* unrot_cos, const float* unrot_sin, cudaStream_t st) {
    return launch_attn<float>(out, q, q_stride, kcache, vcache, tables, max_pages, tok_seq, tok_pos, n_tokens, H, G, dk,
                              dv, window, scale, cap, sinks, unrot_cos, unrot_sin, st);
}
int oe_attn_split_bf16(bf16* out, const bf16* q, long long q_stride, const bf16* kcache, const bf16* vcache,
                       const int* tables, int max_pages, const int* tok_seq, const int* tok_pos, int n_tokens, int H,
                       int G, int dk, int dv, int window, float scale, float cap, const float* sinks,
                       const float* unrot_cos, const float* unrot_sin, cudaStream_t st) {
    return launch_attn<bf16>(out, q, q_stride, kcache, vcache, tables, max_pages, tok_seq, tok_pos, n_tokens, H, G, dk,
                             dv, window, scale, cap, sinks, unrot_cos, unrot_sin, st);
}
}
