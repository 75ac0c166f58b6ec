// Attention over a cache of latents: per token the cache keeps one row [r + rd]: the normed latent c (r values) and,
// when rd > 0, one turned key part shared by all heads.  Every head's key is [Wuk_h c | kr] and its value Wuv_h c, so
// with the query taken through Wuk_h first (qa_h = Wuk_h^T q_h, r values) the score is qa_h . c + qr_h . kr and the
// head's output is Wuv_h (sum_j p_j c_j): all heads read the same cache rows, and keys and values are never expanded.
//
//   latent_write    per token: c = d[:r] / sqrt(mean(d[:r]^2) + eps) * w; kr = d[r:] with the pairs (2i, 2i+1),
//                   i < dims/2, turned by float(position) * freq[i]; both go to the token's cache row (unless the layer
//                   reads another layer's cache).  The last rd dimensions of every query head are turned the same way
//                   and written behind the r absorbed dimensions of the head's row in `qfull` [T, H, r + rd].
//   attn_latent     one warp per (token, head): scores over keys 0 .. pos in chunks of 32 keys at absolute multiples
//                   of 32 (online softmax, float32), output sum_j p_j c_j [r].  A token's result does not depend on
//                   how the step was cut or batched.
//   head_matmul     out[t, h, :] = W_h a[t, h, :] for every head at once, for a handful of tokens (the weights are
//                   streamed once; a warp per weight row, up to 16 tokens' sums in registers); out may be float32.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_R = 512;          // the largest latent

__device__ __forceinline__ long long latent_row(const int* __restrict__ table_row, int pos, int R) {
    const int page = table_row[pos / OE_PAGE];
    if (page < 0) return -1;
    return ((long long)page * OE_PAGE + (pos % OE_PAGE)) * R;
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_write_kernel(const float* d, long long ldd, const float* __restrict__ w, float eps, const T* q, long long ldq,
                    T* qfull, const float* __restrict__ freq, int dims, T* cache, const int* __restrict__ tables,
                    int max_pages, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, int H, int dk, int r,
                    int rd, int write_cache) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    if (b < 0) return;
    const int pos = tok_pos[t];
    const int R = r + rd;
    const float fpos = (float)pos;
    if (write_cache) {
        const float* dr = d + (size_t)t * ldd;
        float ss = 0.f;
        for (int i = threadIdx.x; i < r; i += blockDim.x) { const float v = dr[i]; ss = fmaf(v, v, ss); }
        ss = block_sum(ss, red);
        const long long off = latent_row(tables + (size_t)b * max_pages, pos, R);
        if (off >= 0) {
            const float s = 1.f / sqrtf(ss / (float)r + eps);
            T* row = cache + off;
            for (int i = threadIdx.x; i < r; i += blockDim.x) row[i] = from_f32<T>((dr[i] * s) * w[i]);
            for (int i = threadIdx.x; i < rd; i += blockDim.x) {
                float out;
                if (i < dims) {
                    const int p = i >> 1;
                    float sn, cs;
                    sincosf(fpos * freq[p], &sn, &cs);
                    const float u = dr[r + 2 * p], v = dr[r + 2 * p + 1];
                    out = (i & 1) ? v * cs + u * sn : u * cs - v * sn;
                } else {
                    out = dr[r + i];
                }
                row[r + i] = from_f32<T>(out);
            }
        }
    }
    for (int e = threadIdx.x; e < H * rd; e += blockDim.x) {
        const int hh = e / rd, i = e % rd;
        const T* src = q + (size_t)t * ldq + (size_t)hh * (dk + rd) + dk;
        float out;
        if (i < dims) {
            const int p = i >> 1;
            float sn, cs;
            sincosf(fpos * freq[p], &sn, &cs);
            const float u = to_f32(src[2 * p]), v = to_f32(src[2 * p + 1]);
            out = (i & 1) ? v * cs + u * sn : u * cs - v * sn;
        } else {
            out = to_f32(src[i]);
        }
        qfull[((size_t)t * H + hh) * R + r + i] = from_f32<T>(out);
    }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_latent_kernel(T* out, const T* qfull, const T* cache, const int* __restrict__ tables, int max_pages,
                   const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, int n_tokens, int H, int r, int rd,
                   float scale) {
    extern __shared__ float qs_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const int R = r + rd;
    float* qs = qs_all + warp * R;
    T* o = out + ((size_t)t * H + h) * r;
    const int b = tok_seq[t];
    if (b < 0) {
        for (int i = lane; i < r; i += 32) o[i] = from_f32<T>(0.f);
        return;
    }
    const int pos = tok_pos[t];
    const int* trow = tables + (size_t)b * max_pages;
    const T* qr = qfull + ((size_t)t * H + h) * R;
    for (int i = lane; i < R; i += 32) qs[i] = to_f32(qr[i]);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[MAX_R / 32];
#pragma unroll
    for (int i = 0; i < MAX_R / 32; i++) acc[i] = 0.f;

    for (int c0 = 0; c0 <= pos; c0 += 32) {
        const int key = c0 + lane;
        float s = -INFINITY;
        if (key <= pos) {
            const long long off = latent_row(trow, key, R);
            if (off >= 0) {
                const T* kr = cache + off;
                float dot = 0.f;
                for (int i = 0; i < R; i++) dot = fmaf(qs[i], to_f32(kr[i]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float alpha = expf(m - m_new);
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_R / 32; i++) acc[i] *= alpha;
        const int jmax = (pos - c0 < 31) ? pos - c0 : 31;
        for (int j = 0; j <= jmax; j++) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long voff = latent_row(trow, c0 + j, R);
            if (voff < 0) continue;
            const T* vr = cache + voff;
#pragma unroll
            for (int i = 0; i < MAX_R / 32; i++) {
                const int dd = lane + 32 * i;
                if (dd < r) acc[i] = fmaf(pj, to_f32(vr[dd]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < MAX_R / 32; i++) {
        const int dd = lane + 32 * i;
        if (dd < r) o[dd] = from_f32<T>(acc[i] * inv);
    }
}

// grid (rows of W_h in groups of 8, heads, tokens in groups of 16); a warp per weight row, lanes over k.
constexpr int HM_TOK = 16;
template <typename T, typename TO>
__global__ void __launch_bounds__(256)
head_matmul_kernel(TO* out, long long ldo, long long out_hs, const T* a, long long lda, long long a_hs,
                   const T* __restrict__ w, int n_tokens, int N, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp, h = blockIdx.y, t0 = blockIdx.z * HM_TOK;
    pdl_launch_dependents();
    pdl_wait();
    if (n >= N) return;
    const int nt = min(HM_TOK, n_tokens - t0);
    const T* wr = w + ((size_t)h * N + n) * K;
    float acc[HM_TOK];
#pragma unroll
    for (int i = 0; i < HM_TOK; i++) acc[i] = 0.f;
    for (int kk = lane; kk < K; kk += 32) {
        const float wv = to_f32(wr[kk]);
#pragma unroll
        for (int i = 0; i < HM_TOK; i++)
            if (i < nt) acc[i] = fmaf(wv, to_f32(a[(size_t)(t0 + i) * lda + (size_t)h * a_hs + kk]), acc[i]);
    }
#pragma unroll
    for (int i = 0; i < HM_TOK; i++) {
        if (i < nt) {
            const float v = warp_sum(acc[i]);
            if (lane == 0) out[(size_t)(t0 + i) * ldo + (size_t)h * out_hs + n] = from_f32<TO>(v);
        }
    }
}

template <typename T>
int launch_write(const float* d, long long ldd, const float* w, float eps, const T* q, long long ldq, T* qfull,
                 const float* freq, int dims, T* cache, const int* tables, int max_pages, const int* tok_seq,
                 const int* tok_pos, int n_tokens, int H, int dk, int r, int rd, int write_cache, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (r < 1 || rd < 0 || dims < 0 || dims % 2 || dims > rd || H < 1 || dk < 0) return OE_ERR_UNSUPPORTED;
    return oe_launch(latent_write_kernel<T>, dim3(n_tokens), dim3(128), 0, st, d, ldd, w, eps, q, ldq, qfull, freq, dims, cache,
                     tables, max_pages, tok_seq, tok_pos, H, dk, r, rd, write_cache);
}

template <typename T>
int launch_attn(T* out, const T* qfull, const T* cache, const int* tables, int max_pages, const int* tok_seq,
                const int* tok_pos, int n_tokens, int H, int r, int rd, float scale, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (r < 1 || r > MAX_R || rd < 0 || H < 1) return OE_ERR_UNSUPPORTED;
    const size_t smem = (size_t)WARPS * (r + rd) * sizeof(float);
    if (smem > 48 * 1024) return OE_ERR_UNSUPPORTED;
    const long long items = (long long)n_tokens * H;
    const long long blocks = (items + WARPS - 1) / WARPS;
    if (blocks > 2147483647LL) return OE_ERR_UNSUPPORTED;
    return oe_launch(attn_latent_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), smem, st, out, qfull, cache, tables,
                     max_pages, tok_seq, tok_pos, n_tokens, H, r, rd, scale);
}

template <typename T, typename TO>
int launch_hm(TO* out, long long ldo, long long out_hs, const T* a, long long lda, long long a_hs, const T* w, int n_tokens,
              int H, int N, int K, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (H < 1 || H > 65535 || N < 1 || K < 1) return OE_ERR_UNSUPPORTED;
    const int tz = (n_tokens + HM_TOK - 1) / HM_TOK;
    if (tz > 65535) return OE_ERR_UNSUPPORTED;
    return oe_launch(head_matmul_kernel<T, TO>, dim3((N + 7) / 8, H, tz), dim3(256), 0, st, out, ldo, out_hs, a, lda, a_hs, w,
                     n_tokens, N, K);
}

}  // namespace

extern "C" {
int oe_latent_write_f32(const float* d, long long ldd, const float* w, float eps, const float* q, long long ldq, float* qfull,
                        const float* freq, int dims, float* cache, const int* tables, int max_pages, const int* tok_seq,
                        const int* tok_pos, int n_tokens, int H, int dk, int r, int rd, int write_cache, cudaStream_t st) {
    return launch_write<float>(d, ldd, w, eps, q, ldq, qfull, freq, dims, cache, tables, max_pages, tok_seq, tok_pos, n_tokens,
                               H, dk, r, rd, write_cache, st);
}
int oe_latent_write_bf16(const float* d, long long ldd, const float* w, float eps, const bf16* q, long long ldq, bf16* qfull,
                         const float* freq, int dims, bf16* cache, const int* tables, int max_pages, const int* tok_seq,
                         const int* tok_pos, int n_tokens, int H, int dk, int r, int rd, int write_cache, cudaStream_t st) {
    return launch_write<bf16>(d, ldd, w, eps, q, ldq, qfull, freq, dims, cache, tables, max_pages, tok_seq, tok_pos, n_tokens,
                              H, dk, r, rd, write_cache, st);
}
int oe_attn_latent_f32(float* out, const float* qfull, const float* cache, const int* tables, int max_pages,
                       const int* tok_seq, const int* tok_pos, int n_tokens, int H, int r, int rd, float scale,
                       cudaStream_t st) {
    return launch_attn<float>(out, qfull, cache, tables, max_pages, tok_seq, tok_pos, n_tokens, H, r, rd, scale, st);
}
int oe_attn_latent_bf16(bf16* out, const bf16* qfull, const bf16* cache, const int* tables, int max_pages,
                        const int* tok_seq, const int* tok_pos, int n_tokens, int H, int r, int rd, float scale,
                        cudaStream_t st) {
    return launch_attn<bf16>(out, qfull, cache, tables, max_pages, tok_seq, tok_pos, n_tokens, H, r, rd, scale, st);
}
int oe_head_matmul_f32(float* out, long long ldo, long long out_hs, const float* a, long long lda, long long a_hs,
                       const float* w, int n_tokens, int H, int N, int K, cudaStream_t st) {
    return launch_hm<float, float>(out, ldo, out_hs, a, lda, a_hs, w, n_tokens, H, N, K, st);
}
int oe_head_matmul_bf16(bf16* out, long long ldo, long long out_hs, const bf16* a, long long lda, long long a_hs,
                        const bf16* w, int n_tokens, int H, int N, int K, cudaStream_t st) {
    return launch_hm<bf16, bf16>(out, ldo, out_hs, a, lda, a_hs, w, n_tokens, H, N, K, st);
}
int oe_head_matmul_bf16_f32(float* out, long long ldo, long long out_hs, const bf16* a, long long lda, long long a_hs,
                            const bf16* w, int n_tokens, int H, int N, int K, cudaStream_t st) {
    return launch_hm<bf16, float>(out, ldo, out_hs, a, lda, a_hs, w, n_tokens, H, N, K, st);
}
}
