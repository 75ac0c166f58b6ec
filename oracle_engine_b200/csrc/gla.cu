// Gated linear attention with a decay per key channel and token: per sequence and head a matrix S [dk, dv],
//
//   alpha_t = sigmoid(z_t + b)^(1/tau) = exp(-softplus(-(z_t + b)) / tau)            [dk]
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T;      o_t = S_t^T (q_t * q_scale)          (the read-out sees the new state)
//
// everything in float32.  gla_scan walks a step's tokens of one sequence in order, whatever their number: a prompt,
// a piece of one and a single token run the same instructions in the same order, so the cut of a sequence into steps
// changes no bit.  Column j of a head's S belongs to 8 adjacent lanes, lane l keeping rows l, l + 8, ... in registers
// for all tokens of the step; the vectors every column needs (q, k, alpha) go through shared memory a few tokens at
// a time.  grid (heads x column tiles of 32, sequences).
//
// A long prompt in segments (oe_gla_scan_segments): the recurrence is linear in the state, so a sequence's tokens are cut
// into segments of seg_len that run side by side.  Pass 1 walks every segment but a sequence's last from a zero state
// and keeps its end state L_g and the product P_g of its decays; gla_join_kernel then makes every segment's true
// entering state, E_0 = S, E_(g+1) = diag(P_g) E_g + L_g; pass 2 walks every segment from its E_g and writes the
// outputs, the sequence's last segment also the state.  The sums are the same as in one walk up to their order (a
// rounding), which is why the path whose every bit is pinned to one order (float32 serving) does not take it.
#include "common.cuh"

namespace {

constexpr int L = 8;            // lanes per column
constexpr int COLS = 32;        // columns per block
constexpr int CHUNK = 8;        // tokens staged at once

// MODE 0: a sequence's tokens of the step in one walk.  MODE 1 and 2: the two passes over segments (grid z).
template <int PER, int MODE>
__global__ void __launch_bounds__(COLS * L)
gla_scan_kernel(float* o, float* state, const float* q, const float* k, const float* v, long long stride,
                const float* z, long long ldz, const float* __restrict__ bias, const int* __restrict__ seq_slot,
                const int* __restrict__ cu_q, int H, int dk, int dv, float q_scale, float inv_tau, int seg_len,
                float* seg_state, float* seg_decay) {
    extern __shared__ float stage[];          // [CHUNK][3][dk] then [CHUNK][COLS]
    pdl_launch_dependents();
    pdl_wait();
    const int tiles = (dv + COLS - 1) / COLS;
    const int h = blockIdx.x / tiles, col0 = (blockIdx.x % tiles) * COLS, b = blockIdx.y;
    const int slot = seq_slot[b];
    const int row0 = cu_q[b];
    int n = cu_q[b + 1] - row0;
    if (slot < 0 || n <= 0) return;
    int first = 0;
    bool last = true;
    const int g = MODE ? blockIdx.z : 0, n_seg = MODE ? gridDim.z : 1;
    if (MODE) {
        first = g * seg_len;
        if (first >= n) return;
        last = first + seg_len >= n;
        if (MODE == 1 && last) return;                 // nothing comes after it: its end state is made by pass 2
        n = min(n, first + seg_len);
    }
    const int jj = threadIdx.x / L, l = threadIdx.x % L, j = col0 + jj;
    const bool mine = j < dv;
    float* S = state + ((size_t)slot * H + h) * (size_t)dk * dv;
    const float* enter = S;
    if (MODE == 2 && g > 0) enter = seg_state + (((size_t)b * n_seg + g - 1) * H + h) * (size_t)dk * dv;
    float s[PER], prod[MODE == 1 ? PER : 1];
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int row = l + L * i;
        s[i] = (MODE != 1 && mine && row < dk) ? enter[(size_t)row * dv + j] : 0.f;
        if (MODE == 1) prod[i] = 1.f;
    }
    float* sv = stage + CHUNK * 3 * dk;
    for (int c0 = first; c0 < n; c0 += CHUNK) {
        const int cn = min(CHUNK, n - c0);
        for (int e = threadIdx.x; e < cn * dk; e += blockDim.x) {
            const int tt = e / dk, i = e % dk;
            const size_t at = (size_t)(row0 + c0 + tt) * stride + (size_t)h * dk + i;
            float* dst = stage + (size_t)tt * 3 * dk;
            dst[i] = q[at] * q_scale;
            dst[dk + i] = k[at];
            const float x = -(z[(size_t)(row0 + c0 + tt) * ldz + (size_t)h * dk + i] + bias[(size_t)h * dk + i]);
            const float sp = x > 20.f ? x : log1pf(expf(x));              // softplus(-(z + b)) = -log sigmoid(z + b)
            dst[2 * dk + i] = expf(-sp * inv_tau);
        }
        for (int e = threadIdx.x; e < cn * COLS; e += blockDim.x) {
            const int tt = e / COLS, c = e % COLS;
            sv[e] = col0 + c < dv ? v[(size_t)(row0 + c0 + tt) * stride + (size_t)h * dv + col0 + c] : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < cn; tt++) {
            const float* tk = stage + (size_t)tt * 3 * dk;
            const float vj = sv[tt * COLS + jj];
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int i = 0; i < PER; i++) {
                const int row = l + L * i;
                if (row < dk) {
                    s[i] = fmaf(tk[2 * dk + row], s[i], tk[dk + row] * vj);
                    if (MODE == 1) prod[i] *= tk[2 * dk + row];
                    else if (i & 1) a1 = fmaf(tk[row], s[i], a1); else a0 = fmaf(tk[row], s[i], a0);
                }
            }
            if (MODE == 1) continue;
            float acc = a0 + a1;
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (mine && l == 0) o[(size_t)(row0 + c0 + tt) * (size_t)(H * dv) + (size_t)h * dv + j] = acc;
        }
        __syncthreads();
    }
    if (MODE == 1) {
        float* Lg = seg_state + (((size_t)b * n_seg + g) * H + h) * (size_t)dk * dv;
        float* Pg = seg_decay + (((size_t)b * n_seg + g) * H + h) * (size_t)dk;
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int row = l + L * i;
            if (mine && row < dk) Lg[(size_t)row * dv + j] = s[i];
            if (j == 0 && row < dk) Pg[row] = prod[i];
        }
        return;
    }
    if (mine && last) {
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int row = l + L * i;
            if (row < dk) S[(size_t)row * dv + j] = s[i];
        }
    }
}

// The segments' entering states from their end states and decay products, in place: seg_state[b][g] becomes what
// segment g + 1 starts from.  One thread per element of a (sequence, head)'s state; grid (blocks over dk * dv, H, sequences).
__global__ void gla_join_kernel(const float* __restrict__ state, float* seg_state, const float* __restrict__ seg_decay,
                                const int* __restrict__ seq_slot, const int* __restrict__ cu_q, int H, int dk, int dv,
                                int seg_len, int n_seg) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int slot = seq_slot[b], n = cu_q[b + 1] - cu_q[b];
    if (slot < 0 || e >= dk * dv) return;
    float s = state[((size_t)slot * H + h) * (size_t)dk * dv + e];
    for (int g = 0; (g + 1) * seg_len < n; g++) {
        const size_t at = ((size_t)b * n_seg + g) * H + h;
        s = fmaf(seg_decay[at * dk + e / dv], s, seg_state[at * (size_t)dk * dv + e]);
        seg_state[at * (size_t)dk * dv + e] = s;
    }
}

}  // namespace

extern "C" {

// q, k: float32 rows of H*dk, v: rows of H*dv, all with row stride `stride`; z: rows of H*dk with stride ldz; bias [H*dk];
// o [T, H*dv] contiguous; state [slots, H, dk, dv].
int oe_gla_scan(float* o, float* state, const float* q, const float* k, const float* v, long long stride, const float* z,
                long long ldz, const float* bias, const int* seq_slot, const int* cu_q, int n_seqs, int H, int dk, int dv,
                float q_scale, float inv_tau, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || H < 1 || n_seqs > 65535) return OE_ERR_UNSUPPORTED;
    const dim3 grid(H * ((dv + COLS - 1) / COLS), n_seqs), block(COLS * L);
    const size_t smem = (size_t)CHUNK * (3 * dk + COLS) * sizeof(float);
    const int per = (dk + L - 1) / L;
#define OE_GLA(P) \
    if (per <= P) return oe_launch(gla_scan_kernel<P, 0>, grid, block, smem, st, o, state, q, k, v, stride, z, ldz, bias, \
                                   seq_slot, cu_q, H, dk, dv, q_scale, inv_tau, 0, (float*)nullptr, (float*)nullptr);
    OE_GLA(2) OE_GLA(4) OE_GLA(8) OE_GLA(16) OE_GLA(32)
#undef OE_GLA
    return OE_ERR_UNSUPPORTED;
}

// The same result up to the order of the sums, for sequences that bring up to n_seg * seg_len tokens each: segments side
// by side.  seg_state [n_seqs, n_seg, H, dk, dv] and seg_decay [n_seqs, n_seg, H, dk] are scratch.
int oe_gla_scan_segments(float* o, float* state, const float* q, const float* k, const float* v, long long stride,
                         const float* z, long long ldz, const float* bias, const int* seq_slot, const int* cu_q, int n_seqs,
                         int H, int dk, int dv, float q_scale, float inv_tau, int seg_len, int n_seg, float* seg_state,
                         float* seg_decay, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || H < 1 || H > 65535 || n_seqs > 65535 || seg_len < 1 || n_seg < 1 || n_seg > 65535)
        return OE_ERR_UNSUPPORTED;
    const dim3 grid(H * ((dv + COLS - 1) / COLS), n_seqs, n_seg), block(COLS * L);
    const size_t smem = (size_t)CHUNK * (3 * dk + COLS) * sizeof(float);
    const int per = (dk + L - 1) / L;
#define OE_GLA(P) \
    if (per <= P) { \
        int rc = oe_launch(gla_scan_kernel<P, 1>, grid, block, smem, st, o, state, q, k, v, stride, z, ldz, bias, seq_slot, \
                           cu_q, H, dk, dv, q_scale, inv_tau, seg_len, seg_state, seg_decay); \
        if (rc) return rc; \
        rc = oe_launch(gla_join_kernel, dim3((dk * dv + 255) / 256, H, n_seqs), dim3(256), 0, st, (const float*)state, \
                       seg_state, (const float*)seg_decay, seq_slot, cu_q, H, dk, dv, seg_len, n_seg); \
        if (rc) return rc; \
        return oe_launch(gla_scan_kernel<P, 2>, grid, block, smem, st, o, state, q, k, v, stride, z, ldz, bias, seq_slot, \
                         cu_q, H, dk, dv, q_scale, inv_tau, seg_len, seg_state, seg_decay); \
    }
    OE_GLA(2) OE_GLA(4) OE_GLA(8) OE_GLA(16) OE_GLA(32)
#undef OE_GLA
    return OE_ERR_UNSUPPORTED;
}

}  // extern "C"
