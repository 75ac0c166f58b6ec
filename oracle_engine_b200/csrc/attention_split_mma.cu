// bf16 grouped-query attention on the tensor cores for keys and values with head sizes of their own, read from two
// tensors of the paged cache, with a window and a cap on the scores; prompts (causal, ragged batches), pieces of
// prompts and decoded tokens.  Compiled for one pair of head sizes: -DOE_DK=<key size> -DOE_DV=<value size>,
// multiples of 16 up to 256.
//
// A CTA works on one (sequence, KV head) and a tile of query rows; a row is a (token, query head of the group) pair,
// so the G = H/KVH query heads that share a KV head also share every K/V tile the CTA loads.  Each of the 4 warps
// owns 16 rows.  Key blocks are cache pages (64 keys): a page's K panel [64][dk] and V panel [64][dv] are
// contiguous and are staged in shared memory with cp.async, double buffered.  S = Q K^T and O += P V run on
// mma.sync m16n8k16 (bf16 in, float32 accumulate) with ldmatrix fragments.  Scores are float32: s = scale q.k,
// then s <- cap tanh(s / cap) when cap > 0 (tanh as 1 - 2 / (exp(2x) + 1)); the softmax is online, in float32.
// Mask: pos - window < key <= pos (window 0: every key up to pos).  Only the pages that hold a tile's visible
// keys are read, so a windowed layer's cost does not grow with the context.
// A step of single tokens may split a sequence's pages over `n_splits` CTAs (grid x): each writes its unnormalised
// sums, maximum and denominator as float32, and attn_split_merge_kernel puts them together in split order.
//
// -DOE_KV_SHARED=1: the values are the first DV columns of the key rows (DV <= DK), one tensor [pages][KVH][64][DK]:
// attention over a cache of latents, where a row [latent | shared key part] is the key of every head and its first
// part the value (csrc/attention_latent.cu).  Only the key panel is staged; P V reads its first DV columns.
#include "common.cuh"

#ifndef OE_DK
#define OE_DK 128
#endif
#ifndef OE_DV
#define OE_DV 128
#endif
#ifndef OE_KV_SHARED
#define OE_KV_SHARED 0
#endif

namespace {

constexpr int DK = OE_DK, DV = OE_DV;
constexpr int BN = OE_PAGE;
constexpr int NWARPS = 4;
constexpr bool KV_SHARED = OE_KV_SHARED != 0;
constexpr int K_ROW = DK * 2 + 16, V_ROW = KV_SHARED ? K_ROW : DV * 2 + 16;      // padded rows: ldmatrix without bank conflicts
constexpr int K_TILE = BN * K_ROW, V_TILE = KV_SHARED ? 0 : BN * V_ROW;
static_assert(!KV_SHARED || DV <= DK, "shared rows: the values are the first DV columns of the keys");
constexpr int KS = DK / 16;
static_assert(DK % 16 == 0 && DK >= 16 && DK <= 256 && DV % 16 == 0 && DV >= 16 && DV <= 256, "head sizes: multiples of 16 up to 256");

struct Args {
    bf16* out;                 // [T, H*DV]
    const bf16* q;             // rows of q_stride elements, head h at h*DK (rotated already)
    long long q_stride;
    const bf16* kcache;        // [pages][KVH][64][DK]
    const bf16* vcache;        // [pages][KVH][64][DV] (not read when the values are part of the key rows)
    const int* tables;         // [B, max_pages]
    int max_pages;
    const int* cu_q;
    const int* seq_start;
    const int* seq_qlen;
    int H, KVH, window;
    float scale, cap;
    int tokens_per_tile;
    int n_splits;              // > 1: every sequence brings one token; grid x is the split
    float* partial;            // [T, H, n_splits, DV + 2] when n_splits > 1
    const float* sinks;        // null, or [H] float32: exp(sinks[h]) joins the softmax's denominator (no key, no value)
    const float* unrot_cos;    // null, or [positions, DV/2] float32 (with unrot_sin): every head's result is turned back by
    const float* unrot_sin;    //   its query's position, pair (m, m + DV/2) by minus the table's angle, before it is stored
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&h;
}

__device__ __forceinline__ void load_page(uint8_t* ks, uint8_t* vs, const Args& a, int page, int kvh) {
    const bf16* kg = a.kcache + ((size_t)page * a.KVH + kvh) * (size_t)(BN * DK);
    const bf16* vg = a.vcache + ((size_t)page * a.KVH + kvh) * (size_t)(BN * DV);
    for (int c = threadIdx.x; c < BN * DK / 8; c += NWARPS * 32)
        cp_async16(ks + (c / (DK / 8)) * K_ROW + (c % (DK / 8)) * 16, kg + (size_t)c * 8);
    if (KV_SHARED) return;
    for (int c = threadIdx.x; c < BN * DV / 8; c += NWARPS * 32)
        cp_async16(vs + (c / (DV / 8)) * V_ROW + (c % (DV / 8)) * 16, vg + (size_t)c * 8);
}

__global__ void __launch_bounds__(NWARPS * 32)
attn_split_mma_kernel(const Args a) {
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.z, kvh = blockIdx.y;
    const int qlen = a.seq_qlen[b];
    if (qlen <= 0) return;
    const int start = a.seq_start[b];
    const int G = a.H / a.KVH;
    const int tpt = a.tokens_per_tile;
    const int split = a.n_splits > 1 ? blockIdx.x : 0;
    const int t0 = a.n_splits > 1 ? 0 : blockIdx.x * tpt;
    if (t0 >= qlen) return;
    const int nt = min(tpt, qlen - t0);
    const int pos_lo = start + t0, pos_hi = start + t0 + nt - 1;
    const int key_lo = a.window > 0 ? max(0, pos_lo - a.window + 1) : 0;
    int j_lo = key_lo / BN, j_hi = pos_hi / BN;
    if (a.n_splits > 1) {
        const int per = (j_hi - j_lo + a.n_splits) / a.n_splits;
        j_lo += split * per;
        j_hi = min(j_hi, j_lo + per - 1);
    }
    const int* trow = a.tables + (size_t)b * a.max_pages;
    const int n_blocks = max(0, j_hi - j_lo + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int row0 = warp * 16 + gid;
    const long long packed0 = a.cu_q[b] + t0;

    if (n_blocks > 0) load_page(smem, smem + K_TILE, a, trow[j_lo], kvh);
    cp_async_commit();

    int tok[2], pos[2], head[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = row0 + i * 8;
        tok[i] = r / G;
        head[i] = kvh * G + r % G;
        valid[i] = tok[i] < nt;
        pos[i] = start + t0 + tok[i];
    }
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (valid[i]) {
                const bf16* qr = a.q + (packed0 + tok[i]) * a.q_stride + (size_t)head[i] * DK + ks * 16 + tig * 2;
                qf[ks][i] = *(const uint32_t*)qr;
                qf[ks][i + 2] = *(const uint32_t*)(qr + 8);
            } else {
                qf[ks][i] = 0u;
                qf[ks][i + 2] = 0u;
            }
        }
    }
    float oacc[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; n++) { oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float LOG2E = 1.4426950408889634f;
    const float two_over_cap = a.cap > 0.f ? 2.f * a.scale / a.cap : 0.f;
    const float cap_log2 = a.cap * LOG2E, scale_log2 = a.scale * LOG2E;

    for (int it = 0; it < n_blocks; it++) {
        const int j = j_lo + it;
        uint8_t* ks_cur = smem + (size_t)(it & 1) * (K_TILE + V_TILE);
        uint8_t* vs_cur = KV_SHARED ? ks_cur : ks_cur + K_TILE;
        if (it + 1 < n_blocks) {
            uint8_t* nxt = smem + (size_t)((it + 1) & 1) * (K_TILE + V_TILE);
            load_page(nxt, nxt + K_TILE, a, trow[j + 1], kvh);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        float sacc[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; n++) { sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f; }
        {
            const int m = lane >> 3, r = lane & 7;
            const uint8_t* kbase = ks_cur + ((m >> 1) * 8 + r) * K_ROW + (m & 1) * 16;
            uint32_t kb[2][BN / 16][4];
#pragma unroll
            for (int np = 0; np < BN / 16; np++) ldmatrix_x4(kb[0][np], kbase + np * 16 * K_ROW);
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                if (ks + 1 < KS) {
#pragma unroll
                    for (int np = 0; np < BN / 16; np++)
                        ldmatrix_x4(kb[(ks + 1) & 1][np], kbase + np * 16 * K_ROW + (ks + 1) * 32);
                }
#pragma unroll
                for (int np = 0; np < BN / 16; np++) {
                    mma_bf16(sacc[2 * np], qf[ks], kb[ks & 1][np][0], kb[ks & 1][np][1]);
                    mma_bf16(sacc[2 * np + 1], qf[ks], kb[ks & 1][np][2], kb[ks & 1][np][3]);
                }
            }
        }
        // scale, cap, mask; scores in units of log2(e) for the exponentials
        float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < BN / 8; n++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = e >> 1;
                const int key = j * BN + n * 8 + tig * 2 + (e & 1);
                const bool ok = valid[i] && key <= pos[i] && (a.window <= 0 || key > pos[i] - a.window);
                float s;
                if (a.cap > 0.f) {
                    const float ex = __expf(sacc[n][e] * two_over_cap);              // exp(2 s / cap)
                    s = cap_log2 * (1.f - __fdividef(2.f, ex + 1.f));
                } else {
                    s = sacc[n][e] * scale_log2;
                }
                s = ok ? s : -INFINITY;
                sacc[n][e] = s;
                rmax[i] = fmaxf(rmax[i], s);
            }
        }
        float alpha[2], m_use[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            rmax[i] = fmaxf(rmax[i], __shfl_xor_sync(0xffffffffu, rmax[i], 1));
            rmax[i] = fmaxf(rmax[i], __shfl_xor_sync(0xffffffffu, rmax[i], 2));
            const float m_new = fmaxf(m_run[i], rmax[i]);
            m_use[i] = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[i] = exp2f(m_run[i] - m_use[i]);
            m_run[i] = m_new;
        }
        float rsum[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < BN / 8; n++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float p = exp2f(sacc[n][e] - m_use[e >> 1]);
                sacc[n][e] = p;
                rsum[e >> 1] += p;
            }
        }
#pragma unroll
        for (int i = 0; i < 2; i++) l_run[i] = l_run[i] * alpha[i] + rsum[i];
#pragma unroll
        for (int n = 0; n < DV / 8; n++) {
            oacc[n][0] *= alpha[0]; oacc[n][1] *= alpha[0];
            oacc[n][2] *= alpha[1]; oacc[n][3] *= alpha[1];
        }
#pragma unroll
        for (int kk = 0; kk < BN / 16; kk++) {
            uint32_t pa[4];
            pa[0] = pack_bf16(sacc[2 * kk][0], sacc[2 * kk][1]);
            pa[1] = pack_bf16(sacc[2 * kk][2], sacc[2 * kk][3]);
            pa[2] = pack_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
            pa[3] = pack_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
            const int m = lane >> 3, r = lane & 7;
            const uint8_t* vbase = vs_cur + (kk * 16 + (m & 1) * 8 + r) * V_ROW + (m >> 1) * 16;
            uint32_t vb[2][4];
            ldmatrix_x4_trans(vb[0], vbase);
#pragma unroll
            for (int dp = 0; dp < DV / 16; dp++) {
                if (dp + 1 < DV / 16) ldmatrix_x4_trans(vb[(dp + 1) & 1], vbase + (dp + 1) * 32);
                mma_bf16(oacc[2 * dp], pa, vb[dp & 1][0], vb[dp & 1][1]);
                mma_bf16(oacc[2 * dp + 1], pa, vb[dp & 1][2], vb[dp & 1][3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; i++) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    if (a.sinks && a.n_splits <= 1) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (!valid[i]) continue;
            const float sk = a.sinks[head[i]] * LOG2E;
            if (m_run[i] == -INFINITY) l_run[i] = 1.f;
            else if (sk <= m_run[i]) l_run[i] += exp2f(sk - m_run[i]);
            else {                                        // the sink is the largest term: rescale to it
                const float f = exp2f(m_run[i] - sk);
                l_run[i] = l_run[i] * f + 1.f;
#pragma unroll
                for (int n = 0; n < DV / 8; n++) { oacc[n][2 * i] *= f; oacc[n][2 * i + 1] *= f; }
            }
        }
    }
    if (a.n_splits > 1) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (!valid[i]) continue;
            float* p = a.partial + (((packed0 + tok[i]) * a.H + head[i]) * a.n_splits + split) * (long long)(DV + 2);
#pragma unroll
            for (int n = 0; n < DV / 8; n++) {
                p[n * 8 + tig * 2] = oacc[n][2 * i];
                p[n * 8 + tig * 2 + 1] = oacc[n][2 * i + 1];
            }
            if (tig == 0) { p[DV] = m_run[i]; p[DV + 1] = l_run[i]; }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        if (!valid[i]) continue;
        const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
        bf16* o = a.out + (packed0 + tok[i]) * (long long)(a.H * DV) + (size_t)head[i] * DV + tig * 2;
        if (a.unrot_cos != nullptr) {
            // column m of the first half and m + DV/2 lie in the same thread: accumulators n and n + DV/16
            const float* cr = a.unrot_cos + (size_t)pos[i] * (DV / 2) + tig * 2;
            const float* sr = a.unrot_sin + (size_t)pos[i] * (DV / 2) + tig * 2;
#pragma unroll
            for (int n = 0; n < DV / 16; n++) {
                const float2 c = *(const float2*)(cr + n * 8), s = *(const float2*)(sr + n * 8);
                const float u0 = oacc[n][2 * i] * inv, u1 = oacc[n][2 * i + 1] * inv;
                const float v0 = oacc[n + DV / 16][2 * i] * inv, v1 = oacc[n + DV / 16][2 * i + 1] * inv;
                *(uint32_t*)(o + n * 8) = pack_bf16(u0 * c.x + v0 * s.x, u1 * c.y + v1 * s.y);
                *(uint32_t*)(o + n * 8 + DV / 2) = pack_bf16(v0 * c.x - u0 * s.x, v1 * c.y - u1 * s.y);
            }
            continue;
        }
#pragma unroll
        for (int n = 0; n < DV / 8; n++)
            *(uint32_t*)(o + n * 8) = pack_bf16(oacc[n][2 * i] * inv, oacc[n][2 * i + 1] * inv);
    }
}

// One block per (token, head): the splits' sums put together in split order.  Maxima are in units of log2(e).
__global__ void __launch_bounds__(128)
attn_split_merge_kernel(bf16* out, const float* partial, int n_splits, const int* __restrict__ seq_qlen, int H,
                        const float* __restrict__ sinks, const float* __restrict__ unrot_cos,
                        const float* __restrict__ unrot_sin, const int* __restrict__ seq_start) {
    pdl_launch_dependents();
    pdl_wait();
    if (seq_qlen[blockIdx.x / H] <= 0) {                 // a padding sequence: nothing was written for it
        for (int d = threadIdx.x; d < DV; d += blockDim.x) out[(size_t)blockIdx.x * DV + d] = __float2bfloat16_rn(0.f);
        return;
    }
    const float* p = partial + (size_t)blockIdx.x * n_splits * (DV + 2);
    // a sink counts as one more split: maximum sinks[h] (in units of log2(e)), denominator 1, no values
    const float sk = sinks ? sinks[blockIdx.x % H] * 1.4426950408889634f : -INFINITY;
    float m = sk;
    for (int s = 0; s < n_splits; s++) m = fmaxf(m, p[(size_t)s * (DV + 2) + DV]);
    float l = sinks ? exp2f(sk - m) : 0.f;
    for (int s = 0; s < n_splits; s++) {
        const float ms = p[(size_t)s * (DV + 2) + DV];
        if (ms != -INFINITY) l += exp2f(ms - m) * p[(size_t)s * (DV + 2) + DV + 1];
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (unrot_cos != nullptr) {
        // the sequence's one token stands at position seq_start; a thread takes a pair (d, d + DV/2) and turns it back
        const size_t at = (size_t)seq_start[blockIdx.x / H] * (DV / 2);
        for (int d = threadIdx.x; d < DV / 2; d += blockDim.x) {
            float u = 0.f, v = 0.f;
            for (int s = 0; s < n_splits; s++) {
                const float ms = p[(size_t)s * (DV + 2) + DV];
                if (ms != -INFINITY) {
                    const float f = exp2f(ms - m);
                    u = fmaf(f, p[(size_t)s * (DV + 2) + d], u);
                    v = fmaf(f, p[(size_t)s * (DV + 2) + d + DV / 2], v);
                }
            }
            u *= inv;
            v *= inv;
            const float c = unrot_cos[at + d], sn = unrot_sin[at + d];
            out[(size_t)blockIdx.x * DV + d] = __float2bfloat16_rn(u * c + v * sn);
            out[(size_t)blockIdx.x * DV + d + DV / 2] = __float2bfloat16_rn(v * c - u * sn);
        }
        return;
    }
    for (int d = threadIdx.x; d < DV; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; s++) {
            const float ms = p[(size_t)s * (DV + 2) + DV];
            if (ms != -INFINITY) acc = fmaf(exp2f(ms - m), p[(size_t)s * (DV + 2) + d], acc);
        }
        out[(size_t)blockIdx.x * DV + d] = __float2bfloat16_rn(acc * inv);
    }
}

}  // namespace

extern "C" {

int oe_attn_split_mma_dims(int* dk, int* dv) { *dk = DK; *dv = DV; return 0; }

// max_qlen: the most tokens any sequence of the step brings (sizes the grid).
int oe_attn_split_mma(bf16* out, const bf16* q, long long q_stride, const bf16* kcache, const bf16* vcache,
                      const int* tables, int max_pages, const int* cu_q, const int* seq_start, const int* seq_qlen,
                      int n_seqs, int max_qlen, int H, int KVH, int window, float scale, float cap, int n_splits,
                      float* partial, const float* sinks, const float* unrot_cos, const float* unrot_sin, cudaStream_t st) {
    if (n_seqs <= 0 || max_qlen <= 0) return 0;
    if (KVH < 1 || H % KVH || H / KVH > NWARPS * 16 || n_seqs > 65535 || KVH > 65535) return OE_ERR_UNSUPPORTED;
    if (n_splits > 1 && (max_qlen != 1 || partial == nullptr)) return OE_ERR_UNSUPPORTED;
    Args a;
    a.out = out; a.q = q; a.q_stride = q_stride; a.kcache = kcache; a.vcache = vcache; a.tables = tables;
    a.max_pages = max_pages; a.cu_q = cu_q; a.seq_start = seq_start; a.seq_qlen = seq_qlen;
    a.H = H; a.KVH = KVH; a.window = window; a.scale = scale; a.cap = cap;
    a.tokens_per_tile = (NWARPS * 16) / (H / KVH);
    a.n_splits = n_splits > 1 ? n_splits : 1;
    a.partial = partial;
    a.sinks = sinks;
    const bool unrot = unrot_cos != nullptr && unrot_sin != nullptr;
    // with several splits the merge turns the result back, not the kernel that writes the parts
    a.unrot_cos = unrot && a.n_splits <= 1 ? unrot_cos : nullptr;
    a.unrot_sin = unrot && a.n_splits <= 1 ? unrot_sin : nullptr;
    const size_t smem = (size_t)2 * (K_TILE + V_TILE);
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_split_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    if (a.n_splits > 1) {
        // every sequence brings one token: row b of out is sequence b's (padding sequences leave theirs alone)
        const int rc = oe_launch(attn_split_mma_kernel, dim3(a.n_splits, KVH, n_seqs), dim3(NWARPS * 32), smem, st, a);
        if (rc) return rc;
        return oe_launch(attn_split_merge_kernel, dim3(n_seqs * H), dim3(128), 0, st, out, (const float*)partial, a.n_splits, seq_qlen, H, sinks,
                         unrot ? unrot_cos : (const float*)nullptr, unrot ? unrot_sin : (const float*)nullptr, seq_start);
    }
    const dim3 grid((max_qlen + a.tokens_per_tile - 1) / a.tokens_per_tile, KVH, n_seqs);
    return oe_launch(attn_split_mma_kernel, grid, dim3(NWARPS * 32), smem, st, a);
}

}  // extern "C"
