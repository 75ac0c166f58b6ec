// Row-wise kernels of a stream that has no statistics in its norms, a hashed second embedding and looped passes.
//
//   dyt_norm            y = tanh(alpha x) * w + b, x float32 (the residual stream), y in the compute type; no mean
//                       and no variance, so a row's value depends on nothing but itself
//   pair_embed          x[t] = table[id_t] * scale + pair[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets], and row
//                       `buckets` of the pair table for a sequence's first token.  The token before a step's first one
//                       is per-sequence state (prev [slots] int32), read here and written by prev_token_update
//   prev_token_update   prev[slot] = the sequence's last token of the step (a launch of its own: pair_embed's blocks
//                       read the state while others would write it)
//   pass_entry_add      x += e + s  (e [rows, D] float32 or null, s [D] float32): what a looped group of layers adds
//                       to the stream before a pass
//   scale_rows          x *= s, float32 in place (a constant on the logits)
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
dyt_norm_kernel(T* y, const float* x, const float* __restrict__ w, const float* __restrict__ b, float alpha, size_t rows,
                int D) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = rows * (size_t)D;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % D);
        y[i] = from_f32<T>(fmaf(tanhf(alpha * x[i]), w[d], b[d]));
    }
}

// 16-byte pieces: D a multiple of 4, aligned pointers
template <typename T>
__global__ void __launch_bounds__(256)
dyt_norm_vec_kernel(T* y, const float* x, const float* __restrict__ w, const float* __restrict__ b, float alpha,
                    size_t rows, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const int n4 = D / 4;
    const size_t total = rows * (size_t)n4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % n4);
        const float4 v = reinterpret_cast<const float4*>(x)[i];
        const float4 g = reinterpret_cast<const float4*>(w)[c];
        const float4 o = reinterpret_cast<const float4*>(b)[c];
        const float r0 = fmaf(tanhf(alpha * v.x), g.x, o.x), r1 = fmaf(tanhf(alpha * v.y), g.y, o.y);
        const float r2 = fmaf(tanhf(alpha * v.z), g.z, o.z), r3 = fmaf(tanhf(alpha * v.w), g.w, o.w);
        if (sizeof(T) == 4) {
            reinterpret_cast<float4*>(y)[i] = make_float4(r0, r1, r2, r3);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
            uint2 pk;
            pk.x = *(uint32_t*)&lo;
            pk.y = *(uint32_t*)&hi;
            reinterpret_cast<uint2*>(y)[i] = pk;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
pair_embed_kernel(float* x, const T* __restrict__ table, const T* __restrict__ pair, const int* __restrict__ ids,
                  const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ cu_q,
                  const int* __restrict__ seq_slot, const int* prev, int D, int vocab, int buckets, long long mul_prev,
                  long long mul_cur, float scale, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* xr = x + (size_t)t * D;
    const int b = tok_seq[t];
    if (id < 0 || id >= vocab || b < 0) {
        if (threadIdx.x == 0 && err && b >= 0) atomicExch(err, 1);
        for (int d = threadIdx.x; d < D; d += blockDim.x) xr[d] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * D;
    if (pair == nullptr) {
        for (int d = threadIdx.x; d < D; d += blockDim.x) xr[d] = to_f32(row[d]) * scale;
        return;
    }
    long long bucket = buckets;                              // a sequence's first token
    if (tok_pos[t] > 0) {
        const int before = t > cu_q[b] ? ids[t - 1] : prev[seq_slot[b]];
        bucket = ((long long)before * mul_prev + (long long)id * mul_cur) % (long long)buckets;
        if (bucket < 0) bucket += buckets;
    }
    const T* prow = pair + (size_t)bucket * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) xr[d] = fmaf(to_f32(row[d]), scale, to_f32(prow[d]));
}

__global__ void prev_token_update_kernel(int* prev, const int* __restrict__ ids, const int* __restrict__ cu_q,
                                         const int* __restrict__ seq_slot, int n_seqs) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_seqs) return;
    const int slot = seq_slot[b];
    const int n = cu_q[b + 1] - cu_q[b];
    if (slot >= 0 && n > 0) prev[slot] = ids[cu_q[b + 1] - 1];
}

__global__ void __launch_bounds__(256)
pass_entry_add_kernel(float* x, const float* e, const float* __restrict__ s, size_t rows, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = rows * (size_t)D;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i];
        if (e) v += e[i];
        x[i] = v + s[i % D];
    }
}

__global__ void __launch_bounds__(256) scale_rows_kernel(float* x, size_t total, float s) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) x[i] *= s;
}

inline unsigned blocks_for(size_t items) {
    size_t blocks = (items + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return (unsigned)(blocks ? blocks : 1);
}

template <typename T>
int launch_dyt(T* y, const float* x, const float* w, const float* b, float alpha, long long rows, int D, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (D < 1) return OE_ERR_UNSUPPORTED;
    if (D % 4 == 0 && !(((uintptr_t)x | (uintptr_t)w | (uintptr_t)b) & 15) && !((uintptr_t)y & (sizeof(T) * 4 - 1)))
        return oe_launch(dyt_norm_vec_kernel<T>, dim3(blocks_for((size_t)rows * (D / 4))), dim3(256), 0, st, y, x, w, b, alpha,
                         (size_t)rows, D);
    return oe_launch(dyt_norm_kernel<T>, dim3(blocks_for((size_t)rows * D)), dim3(256), 0, st, y, x, w, b, alpha, (size_t)rows, D);
}

}  // namespace

extern "C" {

int oe_dyt_norm_f32(float* y, const float* x, const float* w, const float* b, float alpha, long long rows, int D,
                    cudaStream_t st) {
    return launch_dyt<float>(y, x, w, b, alpha, rows, D, st);
}
int oe_dyt_norm_bf16(bf16* y, const float* x, const float* w, const float* b, float alpha, long long rows, int D,
                     cudaStream_t st) {
    return launch_dyt<bf16>(y, x, w, b, alpha, rows, D, st);
}
int oe_pair_embed_f32(float* x, const float* table, const float* pair, const int* ids, const int* tok_seq,
                      const int* tok_pos, const int* cu_q, const int* seq_slot, const int* prev, int n_tokens, int D,
                      int vocab, int buckets, long long mul_prev, long long mul_cur, float scale, int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (pair != nullptr && (buckets < 1 || prev == nullptr)) return OE_ERR_UNSUPPORTED;
    return oe_launch(pair_embed_kernel<float>, dim3(n_tokens), dim3(256), 0, st, x, table, pair, ids, tok_seq, tok_pos, cu_q,
                     seq_slot, prev, D, vocab, buckets, mul_prev, mul_cur, scale, err);
}
int oe_pair_embed_bf16(float* x, const bf16* table, const bf16* pair, const int* ids, const int* tok_seq,
                       const int* tok_pos, const int* cu_q, const int* seq_slot, const int* prev, int n_tokens, int D,
                       int vocab, int buckets, long long mul_prev, long long mul_cur, float scale, int* err, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (pair != nullptr && (buckets < 1 || prev == nullptr)) return OE_ERR_UNSUPPORTED;
    return oe_launch(pair_embed_kernel<bf16>, dim3(n_tokens), dim3(256), 0, st, x, table, pair, ids, tok_seq, tok_pos, cu_q,
                     seq_slot, prev, D, vocab, buckets, mul_prev, mul_cur, scale, err);
}
int oe_prev_token_update(int* prev, const int* ids, const int* cu_q, const int* seq_slot, int n_seqs, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    return oe_launch(prev_token_update_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, st, prev, ids, cu_q, seq_slot, n_seqs);
}
int oe_pass_entry_add(float* x, const float* e, const float* s, long long rows, int D, cudaStream_t st) {
    if (rows <= 0) return 0;
    return oe_launch(pass_entry_add_kernel, dim3(blocks_for((size_t)rows * D)), dim3(256), 0, st, x, e, s, (size_t)rows, D);
}

int oe_scale_rows(float* x, long long total, float s, cudaStream_t st) {
    if (total <= 0) return 0;
    return oe_launch(scale_rows_kernel, dim3(blocks_for((size_t)total)), dim3(256), 0, st, x, (size_t)total, s);
}

}  // extern "C"
