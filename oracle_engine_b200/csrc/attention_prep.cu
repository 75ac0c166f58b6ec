// What an attention with normed, turned queries, keys AND values does around its softmax.
//
//   qkv_norm_rot_write   one warp per (token, head) of the float32 projection row [q: H dk | k: G dk | v: G dv]:
//                        + bias;  q and k heads: / sqrt(mean(.^2) + eps) * weight (a weight of dk values shared by the
//                        heads), then the first `rot` dimensions turned by the token's position (i paired with
//                        i + rot/2, cosine and sine from a float32 table [positions, rot/2]);  v heads: / sqrt(mean(.^2)
//                        + eps) without a weight, then ALL dv dimensions turned by the position (m paired with m + dv/2,
//                        a table [positions, dv/2] of its own).  q goes to a contiguous [T, H dk] tensor of the compute
//                        type, k and v to the token's rows of the paged cache [pages, G, PAGE, dk] / [pages, G, PAGE, dv].
//                        Each of bias, norm, key rotation, value norm and value rotation can be absent.
//   unrotate_heads       every head of o [T, H dv] turned back by its own token's position (angle -pos * f_m), in place:
//                        with values stored turned by the key's position, a softmax-weighted sum turned back by the
//                        query's position depends on the values through relative positions only.
// All arithmetic is float32.
#include "common.cuh"

namespace {

constexpr int MAX_D = 256;
constexpr int WARPS = 4;

struct PrepArgs {
    const float* proj; long long ld;
    const float* qb; const float* kb; const float* vb;        // biases [H dk], [G dk], [G dv] or null
    const float* qw; const float* kw;                          // norm weights [dk] or null (null: no norm of q / k)
    float eps;
    const float* cos_k; const float* sin_k; int rot;           // key rotation table [positions, rot/2]; rot 0: none
    const float* cos_v; const float* sin_v;                    // value rotation table [positions, dv/2] or null
    int v_norm;
    const int* tables; int max_pages;
    const int* tok_seq; const int* tok_pos;
    int n_tokens, H, G, dk, dv;
};

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
qkv_norm_rot_write_kernel(T* q_out, T* kcache, T* vcache, const PrepArgs a) {
    __shared__ float stage[WARPS][MAX_D];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = a.H + 2 * a.G;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)a.n_tokens * heads) return;
    const int t = (int)(item / heads), hh = (int)(item % heads);
    const int b = a.tok_seq[t];
    if (b < 0) return;
    const int pos = a.tok_pos[t];
    const int kind = hh < a.H ? 0 : (hh < a.H + a.G ? 1 : 2);            // q, k, v
    const int head = kind == 0 ? hh : (kind == 1 ? hh - a.H : hh - a.H - a.G);
    const int d = kind == 2 ? a.dv : a.dk;
    const long long col0 = kind == 0 ? (long long)head * a.dk
                         : (kind == 1 ? (long long)a.H * a.dk + (long long)head * a.dk
                                      : (long long)(a.H + a.G) * a.dk + (long long)head * a.dv);
    const float* src = a.proj + (size_t)t * a.ld + col0;
    const float* bias = kind == 0 ? a.qb : (kind == 1 ? a.kb : a.vb);
    const float* w = kind == 0 ? a.qw : (kind == 1 ? a.kw : nullptr);
    const bool normed = kind == 2 ? a.v_norm != 0 : w != nullptr;
    // everything a lane loads is asked for before the sums: the row's values, the bias, the norm weight and the angles
    const int rot = kind == 2 ? (a.cos_v ? a.dv : 0) : a.rot;
    const int half = rot / 2;
    const float* cr = (kind == 2 ? a.cos_v : a.cos_k) + (size_t)pos * half;
    const float* sr = (kind == 2 ? a.sin_v : a.sin_k) + (size_t)pos * half;
    const int page = kind == 0 ? 0 : a.tables[(size_t)b * a.max_pages + pos / OE_PAGE];
    float v[MAX_D / 32], wn[MAX_D / 32], cs[MAX_D / 32], sn[MAX_D / 32];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_D / 32; j++) {
        const int i = lane + 32 * j;
        v[j] = 0.f; wn[j] = 1.f; cs[j] = 1.f; sn[j] = 0.f;
        if (i < d) {
            v[j] = src[i] + (bias ? bias[(kind == 2 ? (long long)head * a.dv : (long long)head * a.dk) + i] : 0.f);
            if (w) wn[j] = w[i];
            if (i < rot) { const int m = i < half ? i : i - half; cs[j] = cr[m]; sn[j] = sr[m]; }
        }
    }
#pragma unroll
    for (int j = 0; j < MAX_D / 32; j++) ss = fmaf(v[j], v[j], ss);
    ss = warp_sum(ss);
    const float s = normed ? 1.f / sqrtf(ss / (float)d + a.eps) : 1.f;
    float* sm = stage[warp];
#pragma unroll
    for (int j = 0; j < MAX_D / 32; j++) {
        const int i = lane + 32 * j;
        v[j] = (v[j] * s) * wn[j];
        if (i < rot) sm[i] = v[j];               // only the turned dimensions need their partner
    }
    __syncwarp();
    T* dst;
    if (kind == 0) {
        dst = q_out + ((size_t)t * a.H + head) * a.dk;
    } else {
        if (page < 0) return;
        dst = (kind == 1 ? kcache : vcache) + (((size_t)page * a.G + head) * OE_PAGE + (pos % OE_PAGE)) * d;
    }
#pragma unroll
    for (int j = 0; j < MAX_D / 32; j++) {
        const int i = lane + 32 * j;
        if (i >= d) continue;
        float r = v[j];
        if (i < half) r = v[j] * cs[j] - sm[i + half] * sn[j];
        else if (i < rot) r = v[j] * cs[j] + sm[i - half] * sn[j];
        dst[i] = from_f32<T>(r);
    }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
unrotate_heads_kernel(T* o, const float* __restrict__ cos_v, const float* __restrict__ sin_v,
                      const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, int n_tokens, int H, int dv) {
    __shared__ float stage[WARPS][MAX_D];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H);
    if (tok_seq[t] < 0) return;
    const int pos = tok_pos[t];
    const int half = dv / 2;
    T* row = o + (size_t)item * dv;
    float* sm = stage[warp];
    for (int i = lane; i < dv; i += 32) sm[i] = to_f32(row[i]);
    __syncwarp();
    const float* cr = cos_v + (size_t)pos * half;
    const float* sr = sin_v + (size_t)pos * half;
    for (int i = lane; i < 2 * half; i += 32) {
        // the turn by -angle: (u, v) -> (u c + v s, v c - u s)
        const float r = i < half ? sm[i] * cr[i] + sm[i + half] * sr[i] : sm[i] * cr[i - half] - sm[i - half] * sr[i - half];
        row[i] = from_f32<T>(r);
    }
}

template <typename T>
int launch_prep(T* q_out, T* kcache, T* vcache, const PrepArgs& a, cudaStream_t st) {
    if (a.n_tokens <= 0) return 0;
    if (a.dk < 1 || a.dk > MAX_D || a.dv < 1 || a.dv > MAX_D || a.H < 1 || a.G < 1 || a.rot < 0 || a.rot % 2 || a.rot > a.dk
        || (a.cos_v && a.dv % 2))
        return OE_ERR_UNSUPPORTED;
    const long long items = (long long)a.n_tokens * (a.H + 2 * a.G);
    const long long blocks = (items + WARPS - 1) / WARPS;
    if (blocks > 2147483647LL) return OE_ERR_UNSUPPORTED;
    return oe_launch(qkv_norm_rot_write_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, st, q_out, kcache, vcache, a);
}

template <typename T>
int launch_unrot(T* o, const float* cos_v, const float* sin_v, const int* tok_seq, const int* tok_pos, int n_tokens, int H,
                 int dv, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (dv < 2 || dv > MAX_D || dv % 2 || H < 1) return OE_ERR_UNSUPPORTED;
    const long long blocks = ((long long)n_tokens * H + WARPS - 1) / WARPS;
    if (blocks > 2147483647LL) return OE_ERR_UNSUPPORTED;
    return oe_launch(unrotate_heads_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, st, o, cos_v, sin_v, tok_seq,
                     tok_pos, n_tokens, H, dv);
}

PrepArgs make_args(const float* proj, long long ld, const float* qb, const float* kb, const float* vb, const float* qw,
                   const float* kw, float eps, const float* cos_k, const float* sin_k, int rot, const float* cos_v,
                   const float* sin_v, int v_norm, const int* tables, int max_pages, const int* tok_seq, const int* tok_pos,
                   int n_tokens, int H, int G, int dk, int dv) {
    PrepArgs a;
    a.proj = proj; a.ld = ld; a.qb = qb; a.kb = kb; a.vb = vb; a.qw = qw; a.kw = kw; a.eps = eps;
    a.cos_k = cos_k; a.sin_k = sin_k; a.rot = (cos_k && sin_k) ? rot : 0; a.cos_v = (cos_v && sin_v) ? cos_v : nullptr;
    a.sin_v = sin_v; a.v_norm = v_norm; a.tables = tables; a.max_pages = max_pages; a.tok_seq = tok_seq; a.tok_pos = tok_pos;
    a.n_tokens = n_tokens; a.H = H; a.G = G; a.dk = dk; a.dv = dv;
    return a;
}

}  // namespace

extern "C" {

int oe_qkv_norm_rot_write_f32(float* q_out, float* kcache, float* vcache, const float* proj, long long ld, const float* qb,
                              const float* kb, const float* vb, const float* qw, const float* kw, float eps,
                              const float* cos_k, const float* sin_k, int rot, const float* cos_v, const float* sin_v,
                              int v_norm, const int* tables, int max_pages, const int* tok_seq, const int* tok_pos,
                              int n_tokens, int H, int G, int dk, int dv, cudaStream_t st) {
    return launch_prep<float>(q_out, kcache, vcache, make_args(proj, ld, qb, kb, vb, qw, kw, eps, cos_k, sin_k, rot, cos_v, sin_v,
                                                               v_norm, tables, max_pages, tok_seq, tok_pos, n_tokens, H, G, dk, dv), st);
}
int oe_qkv_norm_rot_write_bf16(bf16* q_out, bf16* kcache, bf16* vcache, const float* proj, long long ld, const float* qb,
                               const float* kb, const float* vb, const float* qw, const float* kw, float eps,
                               const float* cos_k, const float* sin_k, int rot, const float* cos_v, const float* sin_v,
                               int v_norm, const int* tables, int max_pages, const int* tok_seq, const int* tok_pos,
                               int n_tokens, int H, int G, int dk, int dv, cudaStream_t st) {
    return launch_prep<bf16>(q_out, kcache, vcache, make_args(proj, ld, qb, kb, vb, qw, kw, eps, cos_k, sin_k, rot, cos_v, sin_v,
                                                              v_norm, tables, max_pages, tok_seq, tok_pos, n_tokens, H, G, dk, dv), st);
}
int oe_unrotate_heads_f32(float* o, const float* cos_v, const float* sin_v, const int* tok_seq, const int* tok_pos,
                          int n_tokens, int H, int dv, cudaStream_t st) {
    return launch_unrot<float>(o, cos_v, sin_v, tok_seq, tok_pos, n_tokens, H, dv, st);
}
int oe_unrotate_heads_bf16(bf16* o, const float* cos_v, const float* sin_v, const int* tok_seq, const int* tok_pos,
                           int n_tokens, int H, int dv, cudaStream_t st) {
    return launch_unrot<bf16>(o, cos_v, sin_v, tok_seq, tok_pos, n_tokens, H, dv, st);
}

}  // extern "C"
