// Per-head products on the tensor cores, all heads in one launch:
//
//   out[t, h, n] = sum_k a[t, h, k] * w[h, n, k]            a [T, H, K] and out [T, H, N] views (token and head strides
//                                                           free, last axis contiguous), w [H, N, K] contiguous
//
// bf16 operands, float32 sums, out bf16 or float32.  The products that take a latent attention's queries through the
// key projection and its heads' sums through the value projection (parts/latent_attention.py) have this shape: a
// weight per head, far too small to fill the GPU head by head.
//
// A CTA of 4 warps computes a tile of 64 tokens x 64 outputs of one head; K goes through shared memory in chunks of
// 64 (cp.async, two stages; rows padded by 16 bytes so that ldmatrix meets no bank conflict); each warp owns 16
// tokens and runs mma.sync m16n8k16.  K is a multiple of 16; rows of a and w start on 16-byte boundaries.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 64, NWARPS = 4;
constexpr int ROW = BK * 2 + 16;                     // bytes of a staged row
constexpr int TILE = BM * ROW;                       // BM == BN: the same for a and w
constexpr int STAGE = 2 * TILE;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// rows [row0, row0 + 64) x columns [k0, k0 + 64) of a matrix whose rows are `ld` elements apart; zeros beyond
// n_rows and K
__device__ __forceinline__ void stage_tile(uint8_t* dst, const bf16* src, long long ld, int row0, int n_rows, int k0, int K) {
    for (int c = threadIdx.x; c < BM * (BK / 8); c += NWARPS * 32) {
        const int rr = c / (BK / 8), kk = (c % (BK / 8)) * 8;
        uint8_t* d = dst + rr * ROW + kk * 2;
        if (row0 + rr < n_rows && k0 + kk < K) cp_async16(d, src + (long long)(row0 + rr) * ld + k0 + kk);
        else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
}

template <typename TO>
__global__ void __launch_bounds__(NWARPS * 32)
head_matmul_mma_kernel(TO* out, long long ldo, long long out_hs, const bf16* a, long long lda, long long a_hs, const bf16* w,
                       int T, int N, int K) {
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int n0 = blockIdx.x * BN, h = blockIdx.y, t0 = blockIdx.z * BM;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bf16* ah = a + (long long)h * a_hs;
    const bf16* wh = w + (long long)h * N * K;
    const int chunks = (K + BK - 1) / BK;

    float acc[BN / 8][4];
#pragma unroll
    for (int n = 0; n < BN / 8; n++) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }

    stage_tile(smem, ah, lda, t0, T, 0, K);
    stage_tile(smem + TILE, wh, K, n0, N, 0, K);
    cp_async_commit();
    for (int c = 0; c < chunks; c++) {
        uint8_t* cur = smem + (size_t)(c & 1) * STAGE;
        if (c + 1 < chunks) {
            uint8_t* nxt = smem + (size_t)((c + 1) & 1) * STAGE;
            stage_tile(nxt, ah, lda, t0, T, (c + 1) * BK, K);
            stage_tile(nxt + TILE, wh, K, n0, N, (c + 1) * BK, K);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint8_t* as = cur + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ROW + (lane >> 4) * 16;
        const int m = lane >> 3, r = lane & 7;
        const uint8_t* ws = cur + TILE + ((m >> 1) * 8 + r) * ROW + (m & 1) * 16;
#pragma unroll
        for (int ks = 0; ks < BK / 16; ks++) {
            uint32_t af[4];
            ldmatrix_x4(af, as + ks * 32);
#pragma unroll
            for (int np = 0; np < BN / 16; np++) {
                uint32_t bf[4];
                ldmatrix_x4(bf, ws + np * 16 * ROW + ks * 32);
                mma_bf16(acc[2 * np], af, bf[0], bf[1]);
                mma_bf16(acc[2 * np + 1], af, bf[2], bf[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    const int row = t0 + warp * 16 + (lane >> 2);
#pragma unroll
    for (int n = 0; n < BN / 8; n++) {
        const int col = n0 + n * 8 + (lane & 3) * 2;
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int t = row + half * 8;
            if (t >= T) continue;
            TO* o = out + (long long)t * ldo + (long long)h * out_hs + col;
            if (col < N) o[0] = from_f32<TO>(acc[n][2 * half]);
            if (col + 1 < N) o[1] = from_f32<TO>(acc[n][2 * half + 1]);
        }
    }
}

template <typename TO>
int launch(TO* out, long long ldo, long long out_hs, const bf16* a, long long lda, long long a_hs, const bf16* w, int T, int H,
           int N, int K, cudaStream_t st) {
    if (T <= 0) return 0;
    if (H < 1 || H > 65535 || N < 1 || K < 16 || K % 16 || (lda % 8) || (a_hs % 8) || ((uintptr_t)a % 16) || ((uintptr_t)w % 16))
        return OE_ERR_UNSUPPORTED;
    const int tz = (T + BM - 1) / BM;
    if (tz > 65535) return OE_ERR_UNSUPPORTED;
    return oe_launch(head_matmul_mma_kernel<TO>, dim3((N + BN - 1) / BN, H, tz), dim3(NWARPS * 32), (size_t)2 * STAGE, st, out,
                     ldo, out_hs, a, lda, a_hs, w, T, N, K);
}

}  // namespace

extern "C" {
int oe_head_matmul_mma_bf16(bf16* out, long long ldo, long long out_hs, const bf16* a, long long lda, long long a_hs,
                            const bf16* w, int T, int H, int N, int K, cudaStream_t st) {
    return launch<bf16>(out, ldo, out_hs, a, lda, a_hs, w, T, H, N, K, st);
}
int oe_head_matmul_mma_f32(float* out, long long ldo, long long out_hs, const bf16* a, long long lda, long long a_hs,
                           const bf16* w, int T, int H, int N, int K, cudaStream_t st) {
    return launch<float>(out, ldo, out_hs, a, lda, a_hs, w, T, H, N, K, st);
}
}
