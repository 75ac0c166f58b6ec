// A generalized delta rule: per head and sequence a matrix S [dk, dv] in float32, carried from token to token,
//
//     S <- diag(w) S - (a * u) (u^T S) + k v^T,   o = S^T r,   u = k / sqrt(|k|^2 + 1e-6)
//
// (both terms read the old S), with a decay w and a removal rate a per key channel:
//     w = exp(-c * sigmoid(W2 tanh(z1) + w0)),   a = sigmoid(za + ba).
//
//   gdelta_prepare   one block per (tile of tokens, head): from the float32 projection row (columns of r, k, v, za and z1 at
//                    given offsets) the vectors the scan reads, one packed row [w | u | a u | k | r w] with every
//                    vector padded to DKP values by zeros, then c1 = sum r a u and c2 = r . k.  The small product
//                    with W2 [H dk, rank] is done here, in float32.
//   gdelta_scan      column j of S belongs to 8 adjacent lanes, each keeps PER rows in registers.  Per token, with
//                    su_j = sum_i u_i S_ij and p_j = sum_i (r_i w_i) S_ij from the OLD state (one pass, two sums):
//                        S_ij <- w_i S_ij - (a u)_i su_j + k_i v_j;    o_j = p_j - c1 su_j + c2 v_j
//                    which is S_new^T r written out.  A step's tokens of a sequence are walked in order whatever their
//                    number, so a prompt, a piece and a single token run the same instructions: the cut of a sequence
//                    into steps changes no bit.  The packed rows of the next tokens arrive in shared memory by
//                    asynchronous copies while a chunk is computed.
#include "common.cuh"

namespace {

constexpr int L = 8;                 // lanes per column
constexpr int COLS = 32;             // columns per block
constexpr int TAIL = 4;              // floats behind the five vectors of a packed row: c1, c2, two unused

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// grid (token tiles, heads), 4 warps.  packed [T, H, 5 DKP + TAIL].  A block takes `tile` consecutive tokens of one head,
// a warp one token at a time (its lanes own the head's key channels, lane + 32 e; every sum is a warp's, so the tokens
// of a block do not wait for one another).  With w2_smem the head's rows of W2 come into shared memory once per block
// (transposed, so that the lanes read consecutive words) and serve all its tokens; for a handful of tokens they are
// read where they lie.  Either way a channel's sum runs over the rank in the same order.
constexpr int PREP_WARPS = 4;

// PREP_E: channels a lane owns (1, 2, 4 or 8: head sizes up to 32, 64, 128, 256), a compile-time count so that the loop
// over the rank carries no instruction for channels the head does not have
template <int PREP_E>
__global__ void __launch_bounds__(PREP_WARPS * 32)
gdelta_prepare_kernel(float* packed, const float* proj, long long ld, int off_r, int off_k, int off_a, int off_z1, int rank,
                      const float* __restrict__ w2, const float* __restrict__ w0, const float* __restrict__ a_bias,
                      float decay_coef, const int* __restrict__ tok_seq, int n_tokens, int H, int dk, int DKP, int tile,
                      int w2_smem) {
    extern __shared__ float dyn[];               // tanh(z1) of the tile's tokens [tile][rank], then W2^T of the head [rank][dk | 1]
    pdl_launch_dependents();
    float* z1s = dyn;
    float* w2s = dyn + (size_t)tile * rank;
    const int ws = dk | 1;                       // an odd row length: the transposing stores hit different banks
    const int h = blockIdx.y, t0 = blockIdx.x * tile;
    const int nt = min(tile, n_tokens - t0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (w2_smem) {                               // weights: not written by any kernel, so they may come before the wait
        const float* src = w2 + (size_t)h * dk * rank;
        for (int e = threadIdx.x; e < dk * rank; e += blockDim.x) w2s[(size_t)(e % rank) * ws + e / rank] = src[e];
    }
    pdl_wait();
    for (int e = threadIdx.x; e < nt * rank; e += blockDim.x)
        z1s[e] = tanhf(proj[(size_t)(t0 + e / rank) * ld + off_z1 + e % rank]);
    __syncthreads();
    for (int tt = warp; tt < nt; tt += PREP_WARPS) {
        const int t = t0 + tt;
        if (tok_seq[t] < 0) continue;
        const float* row = proj + (size_t)t * ld;
        const float* z1 = z1s + (size_t)tt * rank;
        float* out = packed + ((size_t)t * H + h) * (size_t)(5 * DKP + TAIL);
        float kk[PREP_E], rr[PREP_E], za[PREP_E], z[PREP_E];
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < PREP_E; e++) {
            const int i = lane + 32 * e;
            kk[e] = rr[e] = za[e] = z[e] = 0.f;
            if (i < dk) {
                kk[e] = row[off_k + h * dk + i];
                rr[e] = row[off_r + h * dk + i];
                za[e] = row[off_a + h * dk + i] + (a_bias ? a_bias[h * dk + i] : 0.f);
                z[e] = w0[h * dk + i];
            }
        }
#pragma unroll
        for (int e = 0; e < PREP_E; e++) ss = fmaf(kk[e], kk[e], ss);
        if (w2_smem) {
            for (int j = 0; j < rank; j++) {
                const float zj = z1[j];
#pragma unroll
                for (int e = 0; e < PREP_E; e++)
                    if (lane + 32 * e < dk) z[e] = fmaf(w2s[(size_t)j * ws + lane + 32 * e], zj, z[e]);
            }
        } else {
#pragma unroll
            for (int e = 0; e < PREP_E; e++) {
                if (lane + 32 * e < dk) {
                    const float* w2r = w2 + (size_t)(h * dk + lane + 32 * e) * rank;
                    for (int j = 0; j < rank; j++) z[e] = fmaf(w2r[j], z1[j], z[e]);
                }
            }
        }
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss + 1e-6f);
        float c1 = 0.f, c2 = 0.f;
#pragma unroll
        for (int e = 0; e < PREP_E; e++) {
            const int i = lane + 32 * e;
            if (i < DKP) {
                float w = 0.f, u = 0.f, au = 0.f, rw = 0.f;
                if (i < dk) {
                    w = expf(-decay_coef * sigmoid_f(z[e]));
                    u = kk[e] * inv;
                    au = sigmoid_f(za[e]) * u;
                    rw = rr[e] * w;
                    c1 = fmaf(rr[e], au, c1);
                    c2 = fmaf(rr[e], kk[e], c2);
                }
                out[i] = w; out[DKP + i] = u; out[2 * DKP + i] = au; out[3 * DKP + i] = kk[e]; out[4 * DKP + i] = rw;
            }
        }
        c1 = warp_sum(c1);
        c2 = warp_sum(c2);
        if (lane == 0) { out[5 * DKP] = c1; out[5 * DKP + 1] = c2; out[5 * DKP + 2] = 0.f; out[5 * DKP + 3] = 0.f; }
    }
}

// Which row of its column lane l keeps in register ii: groups of four consecutive rows dealt round robin over the 8
// lanes, so that the lanes of a column read consecutive 16-byte pieces of a staged vector.
__device__ __forceinline__ int lane_row(int ii, int l) { return (ii >> 2) * 4 * L + 4 * l + (ii & 3); }

// grid (H * column tiles, sequences), 256 threads.  v is read from the projection rows (v_ld floats apart).
template <int PER>
__global__ void __launch_bounds__(COLS * L)
gdelta_scan_kernel(float* o, float* state, const float* packed, const float* v, long long v_ld,
                   const int* __restrict__ seq_slot, const int* __restrict__ cu_q, int H, int dk, int dv, int chunk) {
    extern __shared__ __align__(16) float stage_mem[];
    constexpr int DKP = PER * L;
    constexpr int ROWF = 5 * DKP + TAIL;         // floats of a packed row
    constexpr int TOKF = ROWF + COLS;            // floats of a staged token: the packed row, then the block's v columns
    pdl_launch_dependents();
    pdl_wait();
    const int tiles = (dv + COLS - 1) / COLS;
    const int h = blockIdx.x / tiles, col0 = (blockIdx.x % tiles) * COLS, b = blockIdx.y;
    const int jj = threadIdx.x / L, l = threadIdx.x % L, j = col0 + jj;
    const int slot = seq_slot[b];
    const int row0 = cu_q[b], n = cu_q[b + 1] - row0;
    if (slot < 0 || n <= 0) return;
    const bool mine = j < dv;
    float* S = state + (((size_t)slot * H + h) * dk) * dv;
    float s[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int r = lane_row(i, l);
        s[i] = (mine && r < dk) ? S[(size_t)r * dv + j] : 0.f;
    }
    const bool vvec = (dv % 4 == 0) && (v_ld % 4 == 0) && (((uintptr_t)v) & 15) == 0;
    auto issue = [&](int c0, float* dst) {
        const int cn = min(chunk, n - c0);
        constexpr int P4 = ROWF / 4;
        for (int e = threadIdx.x; e < cn * P4; e += blockDim.x) {
            const int tt = e / P4, r = e % P4;
            cp_async16(dst + tt * TOKF + 4 * r, packed + ((size_t)(row0 + c0 + tt) * H + h) * ROWF + 4 * r);
        }
        if (vvec) {
            for (int e = threadIdx.x; e < cn * (COLS / 4); e += blockDim.x) {
                const int tt = e / (COLS / 4), r = e % (COLS / 4);
                if (col0 + 4 * r < dv)
                    cp_async16(dst + tt * TOKF + ROWF + 4 * r, v + (size_t)(row0 + c0 + tt) * v_ld + (size_t)h * dv + col0 + 4 * r);
            }
        } else {
            for (int e = threadIdx.x; e < cn * COLS; e += blockDim.x) {
                const int tt = e / COLS, r = e % COLS;
                if (col0 + r < dv)
                    cp_async4(dst + tt * TOKF + ROWF + r, v + (size_t)(row0 + c0 + tt) * v_ld + (size_t)h * dv + col0 + r);
            }
        }
        cp_async_commit();
    };
    const int stagef = chunk * TOKF;
    issue(0, stage_mem);
    int buf = 0;
    for (int c0 = 0; c0 < n; c0 += chunk, buf ^= 1) {
        const int cn = min(chunk, n - c0);
        if (c0 + chunk < n) { issue(c0 + chunk, stage_mem + (buf ^ 1) * stagef); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        const float* base = stage_mem + buf * stagef;
#pragma unroll 2
        for (int tt = 0; tt < cn; tt++) {
            const float* tk = base + tt * TOKF;
            const float4* w4 = reinterpret_cast<const float4*>(tk);
            const float4* u4 = reinterpret_cast<const float4*>(tk + DKP);
            const float4* au4 = reinterpret_cast<const float4*>(tk + 2 * DKP);
            const float4* k4 = reinterpret_cast<const float4*>(tk + 3 * DKP);
            const float4* rw4 = reinterpret_cast<const float4*>(tk + 4 * DKP);
            const float c1 = tk[5 * DKP], c2 = tk[5 * DKP + 1];
            const float vj = mine ? tk[ROWF + jj] : 0.f;
            float su[2] = {0.f, 0.f}, p[2] = {0.f, 0.f};
#pragma unroll
            for (int i = 0; i < PER; i += 4) {
                const float4 uu = u4[(i >> 2) * L + l], ww = rw4[(i >> 2) * L + l];
                su[0] = fmaf(uu.x, s[i], su[0]); su[1] = fmaf(uu.y, s[i + 1], su[1]);
                su[0] = fmaf(uu.z, s[i + 2], su[0]); su[1] = fmaf(uu.w, s[i + 3], su[1]);
                p[0] = fmaf(ww.x, s[i], p[0]); p[1] = fmaf(ww.y, s[i + 1], p[1]);
                p[0] = fmaf(ww.z, s[i + 2], p[0]); p[1] = fmaf(ww.w, s[i + 3], p[1]);
            }
            float sut = su[0] + su[1], pt = p[0] + p[1];
#pragma unroll
            for (int sh = 1; sh < L; sh <<= 1) {
                sut += __shfl_xor_sync(0xffffffffu, sut, sh);
                pt += __shfl_xor_sync(0xffffffffu, pt, sh);
            }
#pragma unroll
            for (int i = 0; i < PER; i += 4) {
                const float4 ww = w4[(i >> 2) * L + l], aa = au4[(i >> 2) * L + l], kk = k4[(i >> 2) * L + l];
                s[i] = fmaf(ww.x, s[i], fmaf(-aa.x, sut, kk.x * vj));
                s[i + 1] = fmaf(ww.y, s[i + 1], fmaf(-aa.y, sut, kk.y * vj));
                s[i + 2] = fmaf(ww.z, s[i + 2], fmaf(-aa.z, sut, kk.z * vj));
                s[i + 3] = fmaf(ww.w, s[i + 3], fmaf(-aa.w, sut, kk.w * vj));
            }
            if (mine && l == 0)
                o[(size_t)(row0 + c0 + tt) * (size_t)(H * dv) + (size_t)h * dv + j] = fmaf(c2, vj, fmaf(-c1, sut, pt));
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int r = lane_row(i, l);
        if (mine && r < dk) S[(size_t)r * dv + j] = s[i];
    }
}

template <int PER>
int launch_scan(float* o, float* state, const float* packed, const float* v, long long v_ld, const int* seq_slot,
                const int* cu_q, int n_seqs, int H, int dk, int dv, cudaStream_t st) {
    constexpr int TOKF = 5 * PER * L + TAIL + COLS;
    int chunk = (40 * 1024) / (2 * TOKF * 4);
    if (chunk > 16) chunk = 16;
    if (chunk < 1) chunk = 1;
    const size_t smem = (size_t)2 * chunk * TOKF * sizeof(float);
    static bool attr_set = false;
    if (!attr_set && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(gdelta_scan_kernel<PER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    const int tiles = (dv + COLS - 1) / COLS;
    return oe_launch(gdelta_scan_kernel<PER>, dim3(H * tiles, n_seqs), dim3(COLS * L), smem, st, o, state, packed, v, v_ld,
                     seq_slot, cu_q, H, dk, dv, chunk);
}

int padded_dk(int dk) {
    const int per[] = {4, 8, 12, 16, 24, 32};
    for (int p : per)
        if (dk <= p * L) return p * L;
    return -1;
}

}  // namespace

extern "C" {

// The padded number of key channels of a packed row (a multiple of 32), or -1 if dk is too large.
int oe_gdelta_padded_dk(int dk) { return dk < 1 ? -1 : padded_dk(dk); }

int oe_gdelta_prepare(float* packed, const float* proj, long long ld, int off_r, int off_k, int off_a, int off_z1, int rank,
                      const float* w2, const float* w0, const float* a_bias, float decay_coef, const int* tok_seq,
                      int n_tokens, int H, int dk, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    const int DKP = padded_dk(dk);
    if (DKP < 0 || H < 1 || H > 65535 || rank < 0 || rank > 8192) return OE_ERR_UNSUPPORTED;
    // the sums of a token are formed in the same order whatever the tile, so the tile's size changes no bit
    const int tile = n_tokens >= 1024 ? 16 : (n_tokens >= 64 ? 8 : (n_tokens >= 4 ? PREP_WARPS : 1));
    const size_t w2_bytes = (size_t)(dk | 1) * rank * sizeof(float);
    const int w2_smem = tile >= 8 && w2_bytes <= 64 * 1024 && rank > 0;
    const size_t smem = (size_t)tile * (rank > 0 ? rank : 1) * sizeof(float) + (w2_smem ? w2_bytes : 0);
    const int ne = dk <= 32 ? 1 : (dk <= 64 ? 2 : (dk <= 128 ? 4 : 8));
    auto go = [&](auto kernel) -> int {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        return oe_launch(kernel, dim3((n_tokens + tile - 1) / tile, H), dim3(PREP_WARPS * 32), smem, st, packed, proj, ld, off_r,
                         off_k, off_a, off_z1, rank, w2, w0, a_bias, decay_coef, tok_seq, n_tokens, H, dk, DKP, tile, w2_smem);
    };
    if (ne == 1) return go(gdelta_prepare_kernel<1>);
    if (ne == 2) return go(gdelta_prepare_kernel<2>);
    if (ne == 4) return go(gdelta_prepare_kernel<4>);
    return go(gdelta_prepare_kernel<8>);
}

// o [T, H dv] float32; state [slots, H, dk, dv] float32; packed as gdelta_prepare left it; v: the value columns of the
// projection rows (head h at h dv), v_ld floats from row to row.
int oe_gdelta_scan(float* o, float* state, const float* packed, const float* v, long long v_ld, const int* seq_slot,
                   const int* cu_q, int n_seqs, int H, int dk, int dv, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    const int DKP = padded_dk(dk);
    if (DKP < 0 || dv < 1 || H < 1 || n_seqs > 65535) return OE_ERR_UNSUPPORTED;
    switch (DKP / L) {
        case 4: return launch_scan<4>(o, state, packed, v, v_ld, seq_slot, cu_q, n_seqs, H, dk, dv, st);
        case 8: return launch_scan<8>(o, state, packed, v, v_ld, seq_slot, cu_q, n_seqs, H, dk, dv, st);
        case 12: return launch_scan<12>(o, state, packed, v, v_ld, seq_slot, cu_q, n_seqs, H, dk, dv, st);
        case 16: return launch_scan<16>(o, state, packed, v, v_ld, seq_slot, cu_q, n_seqs, H, dk, dv, st);
        case 24: return launch_scan<24>(o, state, packed, v, v_ld, seq_slot, cu_q, n_seqs, H, dk, dv, st);
        case 32: return launch_scan<32>(o, state, packed, v, v_ld, seq_slot, cu_q, n_seqs, H, dk, dv, st);
    }
    return OE_ERR_UNSUPPORTED;
}

}  // extern "C"
