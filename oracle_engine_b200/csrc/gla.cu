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
#include "common.cuh"

namespace {

constexpr int L = 8;            // lanes per column
constexpr int COLS = 32;        // columns per block
constexpr int CHUNK = 8;        // tokens staged at once

template <int PER>
__global__ void __launch_bounds__(COLS * L)
gla_scan_kernel(float* o, float* state, const float* q, const float* k, const float* v, long long stride,
                const float* z, long long ldz, const float* __restrict__ bias, const int* __restrict__ seq_slot,
                const int* __restrict__ cu_q, int H, int dk, int dv, float q_scale, float inv_tau) {
    extern __shared__ float stage[];          // [CHUNK][3][dk] then [CHUNK][COLS]
    pdl_launch_dependents();
    pdl_wait();
    const int tiles = (dv + COLS - 1) / COLS;
    const int h = blockIdx.x / tiles, col0 = (blockIdx.x % tiles) * COLS, b = blockIdx.y;
    const int slot = seq_slot[b];
    const int row0 = cu_q[b], n = cu_q[b + 1] - row0;
    if (slot < 0 || n <= 0) return;
    const int jj = threadIdx.x / L, l = threadIdx.x % L, j = col0 + jj;
    const bool mine = j < dv;
    float* S = state + ((size_t)slot * H + h) * (size_t)dk * dv;
    float s[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int row = l + L * i;
        s[i] = (mine && row < dk) ? S[(size_t)row * dv + j] : 0.f;
    }
    float* sv = stage + CHUNK * 3 * dk;
    for (int c0 = 0; c0 < n; c0 += CHUNK) {
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
                    if (i & 1) a1 = fmaf(tk[row], s[i], a1); else a0 = fmaf(tk[row], s[i], a0);
                }
            }
            float acc = a0 + a1;
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (mine && l == 0) o[(size_t)(row0 + c0 + tt) * (size_t)(H * dv) + (size_t)h * dv + j] = acc;
        }
        __syncthreads();
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int row = l + L * i;
            if (row < dk) S[(size_t)row * dv + j] = s[i];
        }
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
    if (per <= P) return oe_launch(gla_scan_kernel<P>, grid, block, smem, st, o, state, q, k, v, stride, z, ldz, bias, seq_slot, \
                                   cu_q, H, dk, dv, q_scale, inv_tau);
    OE_GLA(2) OE_GLA(4) OE_GLA(8) OE_GLA(16) OE_GLA(32)
#undef OE_GLA
    return OE_ERR_UNSUPPORTED;
}

}  // extern "C"
