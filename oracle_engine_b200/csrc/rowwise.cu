// Row-wise kernels of layers that norm a sublayer's OUTPUT, gate heads, or rotate interleaved pairs:
//
//   cast_rows          y = x rounded to the compute type (a sublayer that reads the residual stream itself)
//   rmsnorm_add        dst (+)= coef * (y / sqrt(mean(y^2) + eps)) * w        (all float32), optionally with a
//                      copy of the new dst rounded to bfloat16 (the next sublayer's input)
//   relu2              a = max(a, 0)^2 in place
//   tanh_rows          y = tanh(x), float32 in, compute type out
//   head_gate          out[t, h, :] = [o / sqrt(mean(o^2) + eps)] * [w] * act(gate)   per head
//   rot_norm_kv_write  q, k rotated on pairs (2i, 2i+1) of their first `dims` dimensions, then divided
//                      by their root mean square; k goes to the cache's key rows, the k as projected
//                      to its value rows (an attention whose values are its unrotated keys)
//   scaled_add         dst += mult * vec * (c0 y0 + c1 y1)   (all float32; vec one value per column or null,
//                      y1 may be null): a sublayer's output, or the weighted sum of two, times a per-channel
//                      scale and a constant, added to the residual stream
//
// All arithmetic is float32; T is the type of activations and cache.  A row's result depends on
// that row only, and every sum has a fixed order.
#include "common.cuh"

namespace {

template <typename T>
__global__ void cast_rows_kernel(T* y, const float* x, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        y[i] = from_f32<T>(x[i]);
}

// One block per row; up to 4,096 columns a thread keeps its part of the row in registers (float4 pieces).
// accumulate == 0: dst is written, not read.  cast_out: null, or [rows, D] bfloat16 that receives the new dst.
__global__ void __launch_bounds__(256)
rmsnorm_add_kernel(float* dst, const float* y, const float* __restrict__ w, int D, float eps, float coef,
                   int accumulate, bf16* cast_out) {
    __shared__ float red[32];
    constexpr int KEEP = 4;
    pdl_launch_dependents();
    pdl_wait();
    const float* yr = y + (size_t)blockIdx.x * D;
    float* dr = dst + (size_t)blockIdx.x * D;
    bf16* cr = cast_out ? cast_out + (size_t)blockIdx.x * D : nullptr;
    const bool vec = (D % 4 == 0) && D <= KEEP * 4 * 256 && !(((uintptr_t)y | (uintptr_t)dst | (uintptr_t)w) & 15);
    if (vec) {
        const int n4 = D / 4;
        float4 keep[KEEP];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < KEEP; j++) {
            const int i = threadIdx.x + j * 256;
            keep[j] = i < n4 ? reinterpret_cast<const float4*>(yr)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += keep[j].x * keep[j].x + keep[j].y * keep[j].y + keep[j].z * keep[j].z + keep[j].w * keep[j].w;
        }
        ss = block_sum(ss, red);
        const float s = 1.f / sqrtf(ss / (float)D + eps);
#pragma unroll
        for (int j = 0; j < KEEP; j++) {
            const int i = threadIdx.x + j * 256;
            if (i < n4) {
                const float4 g = reinterpret_cast<const float4*>(w)[i];
                float4 d = accumulate ? reinterpret_cast<float4*>(dr)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                d.x += coef * ((keep[j].x * s) * g.x); d.y += coef * ((keep[j].y * s) * g.y);
                d.z += coef * ((keep[j].z * s) * g.z); d.w += coef * ((keep[j].w * s) * g.w);
                reinterpret_cast<float4*>(dr)[i] = d;
                if (cr) {
                    cr[4 * i] = __float2bfloat16_rn(d.x); cr[4 * i + 1] = __float2bfloat16_rn(d.y);
                    cr[4 * i + 2] = __float2bfloat16_rn(d.z); cr[4 * i + 3] = __float2bfloat16_rn(d.w);
                }
            }
        }
        return;
    }
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) { const float v = yr[d]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float s = 1.f / sqrtf(ss / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = (accumulate ? dr[d] : 0.f) + coef * ((yr[d] * s) * w[d]);
        dr[d] = v;
        if (cr) cr[d] = __float2bfloat16_rn(v);
    }
}

template <typename T>
__global__ void relu2_kernel(T* a, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f32(a[i]), 0.f);
        a[i] = from_f32<T>(v * v);
    }
}

template <typename T>
__global__ void tanh_rows_kernel(T* y, const float* x, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        y[i] = from_f32<T>(tanhf(x[i]));
}

__device__ __forceinline__ float act_gate(float g, int act) {
    const float sg = 1.f / (1.f + expf(-g));
    return act == 0 ? sg : g * sg;                 // 0: sigmoid, 1: silu
}

// One warp per (token, head).  wmode 0: no weight, 1: w[dv] shared by the heads, 2: w[H * dv].
template <typename TI, typename T>
__global__ void __launch_bounds__(128)
head_gate_kernel(T* out, const TI* o, long long o_stride, const TI* gate, long long g_stride,
                 const float* __restrict__ w, int n_tokens, int H, int dv, int norm, int wmode, int act, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const TI* orow = o + (size_t)t * o_stride + (size_t)h * dv;
    const TI* grow = gate + (size_t)t * g_stride + (size_t)h * dv;
    T* dst = out + ((size_t)t * H + h) * dv;
    float s = 1.f;
    if (norm) {
        float ss = 0.f;
        for (int d = lane; d < dv; d += 32) { const float v = to_f32(orow[d]); ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        s = 1.f / sqrtf(ss / (float)dv + eps);
    }
    for (int d = lane; d < dv; d += 32) {
        float v = to_f32(orow[d]) * s;
        if (wmode == 1) v *= w[d];
        else if (wmode == 2) v *= w[(size_t)h * dv + d];
        dst[d] = from_f32<T>(v * act_gate(to_f32(grow[d]), act));
    }
}

constexpr int MAX_PAIRS = 4;        // pairs a lane keeps: head sizes up to 256

// One warp per (token, head), heads 0 .. H-1 the queries and H .. H+KVH-1 the keys of the row
// [q heads | k heads | ...] of `qk`.  The angle of pair i at position p is float(p) * inv_freq[i].
template <typename T>
__global__ void __launch_bounds__(128)
rot_norm_kv_write_kernel(T* qk, long long row_stride, const float* __restrict__ inv_freq, int rot_dims,
                         T* cache, const int* __restrict__ tables, int max_pages,
                         const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                         int n_tokens, int H, int KVH, int hd, float eps, int has_kv) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int heads = H + (has_kv ? KVH : 0);
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item % heads);
    const int b = tok_seq[t];
    if (b < 0) return;
    const int pos = tok_pos[t];
    T* src = qk + (size_t)t * row_stride + (size_t)h * hd;
    float u[MAX_PAIRS], v[MAX_PAIRS], ru[MAX_PAIRS], rv[MAX_PAIRS];
    float ss = 0.f;
    const int half = hd / 2;
#pragma unroll
    for (int j = 0; j < MAX_PAIRS; j++) {
        const int i = lane + 32 * j;
        u[j] = v[j] = ru[j] = rv[j] = 0.f;
        if (i < half) {
            u[j] = to_f32(src[2 * i]);
            v[j] = to_f32(src[2 * i + 1]);
            if (2 * i < rot_dims) {
                float sn, cs;
                sincosf((float)pos * inv_freq[i], &sn, &cs);
                ru[j] = u[j] * cs - v[j] * sn;
                rv[j] = v[j] * cs + u[j] * sn;
            } else {
                ru[j] = u[j];
                rv[j] = v[j];
            }
            ss = fmaf(ru[j], ru[j], ss);
            ss = fmaf(rv[j], rv[j], ss);
        }
    }
    ss = warp_sum(ss);
    const float s = 1.f / sqrtf(ss / (float)hd + eps);
    T* key_dst = src;
    T* val_dst = nullptr;
    if (h >= H) {
        const int* trow = tables + (size_t)b * max_pages;
        const long long ko = page_row_offset(trow, pos, 0, h - H, KVH, hd);
        const long long vo = page_row_offset(trow, pos, 1, h - H, KVH, hd);
        if (ko < 0) return;
        key_dst = cache + ko;
        val_dst = cache + vo;
    }
#pragma unroll
    for (int j = 0; j < MAX_PAIRS; j++) {
        const int i = lane + 32 * j;
        if (i < half) {
            key_dst[2 * i] = from_f32<T>(ru[j] * s);
            key_dst[2 * i + 1] = from_f32<T>(rv[j] * s);
            if (val_dst) {
                val_dst[2 * i] = from_f32<T>(u[j]);
                val_dst[2 * i + 1] = from_f32<T>(v[j]);
            }
        }
    }
}

inline int flat_blocks(size_t total) {
    const size_t b = (total + 255) / 256;
    return (int)(b < 148 * 16 ? b : 148 * 16);
}

template <typename TI, typename T>
int head_gate_launch(T* out, const TI* o, long long o_stride, const TI* gate, long long g_stride, const float* w,
                     int n_tokens, int H, int dv, int norm, int wmode, int act, float eps, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || dv <= 0 || (wmode != 0 && w == nullptr)) return OE_ERR_UNSUPPORTED;
    const long long items = (long long)n_tokens * H;
    const long long blocks = (items + 3) / 4;
    if (blocks > 2147483647LL) return OE_ERR_UNSUPPORTED;
    return oe_launch(head_gate_kernel<TI, T>, dim3((unsigned)blocks), dim3(128), 0, st, out, o, o_stride, gate, g_stride, w,
                     n_tokens, H, dv, norm, wmode, act, eps);
}

template <typename T>
int rot_norm_launch(T* qk, long long row_stride, const float* inv_freq, int rot_dims, T* cache, const int* tables,
                    int max_pages, const int* tok_seq, const int* tok_pos, int n_tokens, int H, int KVH, int hd, float eps,
                    int has_kv, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (hd % 2 || hd > 64 * MAX_PAIRS || rot_dims % 2 || rot_dims < 0 || rot_dims > hd) return OE_ERR_UNSUPPORTED;
    const long long items = (long long)n_tokens * (H + (has_kv ? KVH : 0));
    const long long blocks = (items + 3) / 4;
    if (blocks > 2147483647LL) return OE_ERR_UNSUPPORTED;
    return oe_launch(rot_norm_kv_write_kernel<T>, dim3((unsigned)blocks), dim3(128), 0, st, qk, row_stride, inv_freq, rot_dims,
                     cache, tables, max_pages, tok_seq, tok_pos, n_tokens, H, KVH, hd, eps, has_kv);
}


__global__ void __launch_bounds__(256)
scaled_add_kernel(float* dst, const float* y0, const float* y1, const float* __restrict__ vec, float mult, float c0,
                  float c1, size_t total, int D) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = c0 * y0[i];
        if (y1) v = fmaf(c1, y1[i], v);
        const float sc = vec ? mult * vec[i % D] : mult;
        dst[i] = fmaf(sc, v, dst[i]);
    }
}

}  // namespace

extern "C" {

int oe_scaled_add(float* dst, const float* y0, const float* y1, const float* vec, float mult, float c0, float c1,
                  long long rows, int D, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (D < 1) return OE_ERR_UNSUPPORTED;
    const size_t total = (size_t)rows * D;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return oe_launch(scaled_add_kernel, dim3((unsigned)blocks), dim3(256), 0, st, dst, y0, y1, vec, mult, c0, c1, total, D);
}

int oe_cast_rows_bf16(bf16* y, const float* x, long long total, cudaStream_t st) {
    if (total <= 0) return 0;
    return oe_launch(cast_rows_kernel<bf16>, dim3(flat_blocks((size_t)total)), dim3(256), 0, st, y, x, (size_t)total);
}

int oe_rmsnorm_add(float* dst, const float* y, const float* w, int rows, int D, float eps, float coef, int accumulate,
                   bf16* cast_out, cudaStream_t st) {
    if (rows <= 0) return 0;
    return oe_launch(rmsnorm_add_kernel, dim3(rows), dim3(256), 0, st, dst, y, w, D, eps, coef, accumulate, cast_out);
}

int oe_relu2_f32(float* a, long long total, cudaStream_t st) {
    if (total <= 0) return 0;
    return oe_launch(relu2_kernel<float>, dim3(flat_blocks((size_t)total)), dim3(256), 0, st, a, (size_t)total);
}
int oe_relu2_bf16(bf16* a, long long total, cudaStream_t st) {
    if (total <= 0) return 0;
    return oe_launch(relu2_kernel<bf16>, dim3(flat_blocks((size_t)total)), dim3(256), 0, st, a, (size_t)total);
}

int oe_tanh_rows_f32(float* y, const float* x, long long total, cudaStream_t st) {
    if (total <= 0) return 0;
    return oe_launch(tanh_rows_kernel<float>, dim3(flat_blocks((size_t)total)), dim3(256), 0, st, y, x, (size_t)total);
}
int oe_tanh_rows_bf16(bf16* y, const float* x, long long total, cudaStream_t st) {
    if (total <= 0) return 0;
    return oe_launch(tanh_rows_kernel<bf16>, dim3(flat_blocks((size_t)total)), dim3(256), 0, st, y, x, (size_t)total);
}

// o and gate float32 (a recurrence's read-out and a float32 projection), out of the compute type
int oe_head_gate_f32_f32(float* out, const float* o, long long o_stride, const float* gate, long long g_stride,
                         const float* w, int n_tokens, int H, int dv, int norm, int wmode, int act, float eps, cudaStream_t st) {
    return head_gate_launch<float, float>(out, o, o_stride, gate, g_stride, w, n_tokens, H, dv, norm, wmode, act, eps, st);
}
int oe_head_gate_f32_bf16(bf16* out, const float* o, long long o_stride, const float* gate, long long g_stride,
                          const float* w, int n_tokens, int H, int dv, int norm, int wmode, int act, float eps, cudaStream_t st) {
    return head_gate_launch<float, bf16>(out, o, o_stride, gate, g_stride, w, n_tokens, H, dv, norm, wmode, act, eps, st);
}
// o and gate of the compute type (an attention's output and its gate projection)
int oe_head_gate_bf16_bf16(bf16* out, const bf16* o, long long o_stride, const bf16* gate, long long g_stride,
                           const float* w, int n_tokens, int H, int dv, int norm, int wmode, int act, float eps, cudaStream_t st) {
    return head_gate_launch<bf16, bf16>(out, o, o_stride, gate, g_stride, w, n_tokens, H, dv, norm, wmode, act, eps, st);
}

int oe_rot_norm_kv_write_f32(float* qk, long long row_stride, const float* inv_freq, int rot_dims, float* cache,
                             const int* tables, int max_pages, const int* tok_seq, const int* tok_pos, int n_tokens, int H,
                             int KVH, int hd, float eps, int has_kv, cudaStream_t st) {
    return rot_norm_launch<float>(qk, row_stride, inv_freq, rot_dims, cache, tables, max_pages, tok_seq, tok_pos, n_tokens, H,
                                  KVH, hd, eps, has_kv, st);
}
int oe_rot_norm_kv_write_bf16(bf16* qk, long long row_stride, const float* inv_freq, int rot_dims, bf16* cache,
                              const int* tables, int max_pages, const int* tok_seq, const int* tok_pos, int n_tokens, int H,
                              int KVH, int hd, float eps, int has_kv, cudaStream_t st) {
    return rot_norm_launch<bf16>(qk, row_stride, inv_freq, rot_dims, cache, tables, max_pages, tok_seq, tok_pos, n_tokens, H,
                                 KVH, hd, eps, has_kv, st);
}

}  // extern "C"
