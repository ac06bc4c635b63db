// Recurrent mixers: layers whose memory is a matrix per head and sequence, of fixed size, kept in
// float32 in the state store and carried from step to step.
//
//   short_conv_prepare   the inputs of a gated delta rule from one float32 projection row:
//                        causal convolution over time per channel + silu (q, k, v), unit vectors per
//                        head (q, k), step size beta = sigmoid(.), decay g = exp(-exp(A) softplus(. + dt))
//   conv_state_update    the last taps-1 projection rows of every sequence, kept for the next step
//   delta_rule_scan      S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   token_shift_mix      m_s = h + (h_prev - h) mu_s for several s at once
//   last_rows_to_state   a sequence's last row of the step, kept for the next step
//   decay_scan           o = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T, w = exp(-exp(z + w0))
//
// Both scans give column j of a head's S to a few adjacent threads (each a share of its rows): the columns
// never mix, so the threads keep their column in registers for all tokens of the step, and the vectors
// every column needs (k, q, r, w) go through shared memory a few tokens at a time.  A step's tokens of one sequence are walked in
// order, whatever their number: a prompt, a piece of one and a single token run the same
// instructions in the same order, so the cut of a sequence into steps changes no bit.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;
constexpr int CHUNK = 8;            // tokens whose vectors are staged at once

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// proj row: [q: G*dk | k: G*dk | v: H*dv | gate: H*dv | beta: H | a: H]; one block per token.
// out_qkv row [q | k | v] (C = 2 G dk + H dv), out_gb row [g: H | beta: H].
__global__ void __launch_bounds__(256)
short_conv_prepare_kernel(float* out_qkv, float* out_gb, const float* proj, int P,
                          const float* __restrict__ conv_w, int taps, const float* conv_state,
                          const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                          const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                          const int* __restrict__ cu_q, int G, int H, int dk, int dv, float q_scale) {
    extern __shared__ float act[];              // the token's q and k after convolution and silu
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    if (b < 0) return;
    const int slot = seq_slot[b];
    const int rel = t - cu_q[b];                // index of the token among its sequence's tokens of this step
    const int nqk = 2 * G * dk, C = nqk + H * dv;
    const float* st = conv_state + (size_t)slot * (taps - 1) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < taps; j++) {
            const int r = rel - (taps - 1) + j;
            const float x = r >= 0 ? proj[(size_t)(t - rel + r) * P + c] : st[(size_t)(rel + j) * C + c];
            acc = fmaf(conv_w[(size_t)c * taps + j], x, acc);
        }
        const float y = silu_f(acc);
        if (c < nqk) act[c] = y;
        else out_qkv[(size_t)t * C + c] = y;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int hh = warp; hh < 2 * G; hh += nwarps) {
        const float* a = act + (size_t)hh * dk;
        float ss = 0.f;
        for (int d = lane; d < dk; d += 32) ss = fmaf(a[d], a[d], ss);
        ss = warp_sum(ss);
        const float s = (1.f / sqrtf(ss + 1e-6f)) * (hh < G ? q_scale : 1.f);
        for (int d = lane; d < dk; d += 32) out_qkv[(size_t)t * C + (size_t)hh * dk + d] = a[d] * s;
    }
    const float* row = proj + (size_t)t * P;
    for (int hh = threadIdx.x; hh < H; hh += blockDim.x) {
        const float bt = row[C + H * dv + hh], a = row[C + H * dv + H + hh];
        out_gb[(size_t)t * 2 * H + hh] = expf(-expf(A_log[hh]) * softplus_f(a + dt_bias[hh]));
        out_gb[(size_t)t * 2 * H + H + hh] = 1.f / (1.f + expf(-bt));
    }
}

// One block per sequence; a thread owns whole channels, so it reads a channel's old rows before it writes them.
__global__ void __launch_bounds__(256)
conv_state_update_kernel(float* conv_state, const float* proj, int P, int C, int taps,
                         const int* __restrict__ seq_slot, const int* __restrict__ cu_q) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int slot = seq_slot[b];
    const int row0 = cu_q[b], n = cu_q[b + 1] - row0;
    if (slot < 0 || n <= 0) return;
    float* st = conv_state + (size_t)slot * (taps - 1) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float keep[MAX_TAPS];
#pragma unroll
        for (int i = 0; i < MAX_TAPS; i++) {
            if (i < taps - 1) {
                const int r = n - (taps - 1) + i;
                keep[i] = r >= 0 ? proj[(size_t)(row0 + r) * P + c] : st[(size_t)(n + i) * C + c];
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_TAPS; i++)
            if (i < taps - 1) st[(size_t)i * C + c] = keep[i];
    }
}

// Sum over the L adjacent lanes that share a column (L a power of two up to 8), the same order everywhere.
template <int L>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = 1; o < L; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// grid (H, B).  Column j of S[dk][dv] of head blockIdx.x of sequence blockIdx.y belongs to the L adjacent
// threads j*L .. j*L+L-1; thread l of them keeps rows l*PER .. l*PER+PER-1 in registers (dk = L * per,
// per <= PER).  qkv row [q: G*dk | k: G*dk | v: H*dv], gb row [g: H | beta: H]; o [T, H*dv] float32.
template <int PER, int L>
__global__ void __launch_bounds__(PER >= 64 ? 256 : 512)
delta_rule_scan_kernel(float* o, float* state, const float* qkv, const float* gb,
                       const int* __restrict__ seq_slot, const int* __restrict__ cu_q,
                       int G, int H, int dk, int dv) {
    __shared__ float kq[CHUNK][2][PER * L];
    __shared__ float sc[CHUNK][2];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y, j = threadIdx.x / L, l = threadIdx.x % L;
    const int slot = seq_slot[b];
    const int row0 = cu_q[b], n = cu_q[b + 1] - row0;
    if (slot < 0 || n <= 0) return;
    const int g = h / (H / G);
    const int C = 2 * G * dk + H * dv;
    const int per = dk / L, i0 = l * per;
    const bool mine = j < dv;
    float* S = state + (((size_t)slot * H + h) * dk) * dv;
    float s[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) s[i] = (mine && i < per) ? S[(size_t)(i0 + i) * dv + j] : 0.f;
    for (int c0 = 0; c0 < n; c0 += CHUNK) {
        const int cn = min(CHUNK, n - c0);
        __syncthreads();
        for (int e = threadIdx.x; e < cn * 2 * dk; e += blockDim.x) {
            const int tt = e / (2 * dk), r = e % (2 * dk), which = r / dk, d = r % dk;      // which 0: k, 1: q
            kq[tt][which][d] = qkv[(size_t)(row0 + c0 + tt) * C + (size_t)(which == 0 ? G + g : g) * dk + d];
        }
        if (threadIdx.x < cn * 2) {
            const int tt = threadIdx.x / 2, w = threadIdx.x % 2;
            sc[tt][w] = gb[(size_t)(row0 + c0 + tt) * 2 * H + (size_t)w * H + h];
        }
        __syncthreads();
        for (int tt = 0; tt < cn; tt++) {
            const size_t row = (size_t)(row0 + c0 + tt);
            const float decay = sc[tt][0], beta = sc[tt][1];
            const float v = mine ? qkv[row * C + (size_t)2 * G * dk + (size_t)h * dv + j] : 0.f;
            const float* kk = &kq[tt][0][i0];
            const float* qq = &kq[tt][1][i0];
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < PER; i++)
                if (i < per) { s[i] *= decay; dot = fmaf(kk[i], s[i], dot); }
            dot = lanes_sum<L>(dot);
            const float u = beta * (v - dot);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < PER; i++)
                if (i < per) { s[i] = fmaf(kk[i], u, s[i]); acc = fmaf(qq[i], s[i], acc); }
            acc = lanes_sum<L>(acc);
            if (mine && l == 0) o[row * (size_t)(H * dv) + (size_t)h * dv + j] = acc;
        }
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < PER; i++)
            if (i < per) S[(size_t)(i0 + i) * dv + j] = s[i];
    }
}

// One block per token.  out[s][t][:] = h[t] + (prev - h[t]) * mu[s], prev = the row before in the same
// sequence, or the sequence's kept row (zeros at its start).
template <typename T>
__global__ void __launch_bounds__(256)
token_shift_mix_kernel(T* out, const T* h, const float* __restrict__ mu, const float* prev_state, int n_mix,
                       int n_tokens, int D, const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                       const int* __restrict__ cu_q) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    if (b < 0) return;
    const bool first = t == cu_q[b];
    const float* st = prev_state + (size_t)seq_slot[b] * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float cur = to_f32(h[(size_t)t * D + d]);
        const float prev = first ? st[d] : to_f32(h[(size_t)(t - 1) * D + d]);
        const float diff = prev - cur;
        for (int s = 0; s < n_mix; s++)
            out[((size_t)s * n_tokens + t) * D + d] = from_f32<T>(fmaf(diff, mu[(size_t)s * D + d], cur));
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
last_rows_to_state_kernel(float* state, const T* h, int D, const int* __restrict__ seq_slot,
                          const int* __restrict__ cu_q) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int slot = seq_slot[b];
    const int last = cu_q[b + 1] - 1;
    if (slot < 0 || last < cu_q[b]) return;
    for (int d = threadIdx.x; d < D; d += blockDim.x) state[(size_t)slot * D + d] = to_f32(h[(size_t)last * D + d]);
}

// grid (H, B); column j of S[d][d] belongs to L adjacent threads as in the delta rule's scan.  r, k, v, z:
// float32 rows of H*d with one row stride; u, w0: [H*d].
template <int PER, int L>
__global__ void __launch_bounds__(PER >= 64 ? 256 : 512)
decay_scan_kernel(float* o, float* state, const float* r, const float* k, const float* v, const float* z,
                  long long stride, const float* __restrict__ u, const float* __restrict__ w0,
                  const int* __restrict__ seq_slot, const int* __restrict__ cu_q, int H, int d) {
    __shared__ float vec[CHUNK][4][PER * L];          // per token: 0 r, 1 k, 2 w, 3 u*k
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y, j = threadIdx.x / L, l = threadIdx.x % L;
    const int slot = seq_slot[b];
    const int row0 = cu_q[b], n = cu_q[b + 1] - row0;
    if (slot < 0 || n <= 0) return;
    const int per = d / L, i0 = l * per;
    const bool mine = j < d;
    float* S = state + (((size_t)slot * H + h) * d) * d;
    float s[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) s[i] = (mine && i < per) ? S[(size_t)(i0 + i) * d + j] : 0.f;
    for (int c0 = 0; c0 < n; c0 += CHUNK) {
        const int cn = min(CHUNK, n - c0);
        __syncthreads();
        for (int e = threadIdx.x; e < cn * d; e += blockDim.x) {
            const int tt = e / d, i = e % d;
            const size_t at = (size_t)(row0 + c0 + tt) * stride + (size_t)h * d + i;
            const float kk = k[at];
            vec[tt][0][i] = r[at];
            vec[tt][1][i] = kk;
            vec[tt][2][i] = expf(-expf(z[at] + w0[(size_t)h * d + i]));
            vec[tt][3][i] = u[(size_t)h * d + i] * kk;
        }
        __syncthreads();
        for (int tt = 0; tt < cn; tt++) {
            const size_t row = (size_t)(row0 + c0 + tt);
            const float vj = mine ? v[row * stride + (size_t)h * d + j] : 0.f;
            const float* rr = &vec[tt][0][i0];
            const float* kk = &vec[tt][1][i0];
            const float* ww = &vec[tt][2][i0];
            const float* uk = &vec[tt][3][i0];
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < PER; i++) {
                if (i < per) {
                    acc = fmaf(rr[i], fmaf(uk[i], vj, s[i]), acc);
                    s[i] = fmaf(ww[i], s[i], kk[i] * vj);
                }
            }
            acc = lanes_sum<L>(acc);
            if (mine && l == 0) o[row * (size_t)(H * d) + (size_t)h * d + j] = acc;
        }
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < PER; i++)
            if (i < per) S[(size_t)(i0 + i) * d + j] = s[i];
    }
}

// Lanes per column: the most of 8, 4, 2, 1 that divide the rows, leave each lane 8 rows or more and keep
// the block within 512 threads (256 where a lane keeps 64 rows or more in registers).
inline int lanes_per_column(int rows, int cols) {
    for (int L = 8; L > 1; L >>= 1)
        if (rows % L == 0 && rows / L >= 8 && cols * L <= (rows / L > 32 ? 256 : 512)) return L;
    return 1;
}

inline int round_up_warp(int n) { return (n + 31) / 32 * 32; }

}  // namespace

extern "C" {

int oe_short_conv_prepare(float* out_qkv, float* out_gb, const float* proj, int P, const float* conv_w, int taps,
                          const float* conv_state, const float* A_log, const float* dt_bias, const int* tok_seq,
                          const int* seq_slot, const int* cu_q, int n_tokens, int G, int H, int dk, int dv, float q_scale,
                          cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (taps < 1 || taps > MAX_TAPS || G < 1 || H % G) return OE_ERR_UNSUPPORTED;
    const size_t smem = (size_t)2 * G * dk * sizeof(float);
    if (smem > 200 * 1024) return OE_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(short_conv_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return oe_launch(short_conv_prepare_kernel, dim3(n_tokens), dim3(256), smem, st, out_qkv, out_gb, proj, P, conv_w, taps,
                     conv_state, A_log, dt_bias, tok_seq, seq_slot, cu_q, G, H, dk, dv, q_scale);
}

int oe_conv_state_update(float* conv_state, const float* proj, int P, int C, int taps, const int* seq_slot,
                         const int* cu_q, int n_seqs, cudaStream_t st) {
    if (n_seqs <= 0 || taps <= 1) return 0;
    if (taps > MAX_TAPS) return OE_ERR_UNSUPPORTED;
    return oe_launch(conv_state_update_kernel, dim3(n_seqs), dim3(256), 0, st, conv_state, proj, P, C, taps, seq_slot, cu_q);
}

int oe_delta_rule_scan(float* o, float* state, const float* qkv, const float* gb, const int* seq_slot, const int* cu_q,
                       int n_seqs, int G, int H, int dk, int dv, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || dv > 256 || G < 1 || H % G || n_seqs > 65535) return OE_ERR_UNSUPPORTED;
    const int L = lanes_per_column(dk, dv), per = dk / L;
    const dim3 grid(H, n_seqs), block(round_up_warp(dv * L));
    if (block.x > (per > 32 ? 256u : 512u)) return OE_ERR_UNSUPPORTED;
#define OE_SCAN(PER, LL) \
    if (L == LL && per <= PER) return oe_launch(delta_rule_scan_kernel<PER, LL>, grid, block, 0, st, o, state, qkv, gb, seq_slot, cu_q, G, H, dk, dv);
    OE_SCAN(8, 8) OE_SCAN(16, 8) OE_SCAN(32, 8)
    OE_SCAN(8, 4) OE_SCAN(16, 4) OE_SCAN(32, 4) OE_SCAN(64, 4)
    OE_SCAN(8, 2) OE_SCAN(16, 2) OE_SCAN(32, 2) OE_SCAN(64, 2) OE_SCAN(128, 2)
    OE_SCAN(8, 1) OE_SCAN(16, 1) OE_SCAN(32, 1) OE_SCAN(64, 1) OE_SCAN(128, 1) OE_SCAN(256, 1)
#undef OE_SCAN
    return OE_ERR_UNSUPPORTED;
}

int oe_token_shift_mix_f32(float* out, const float* h, const float* mu, const float* prev_state, int n_mix, int n_tokens,
                           int D, const int* tok_seq, const int* seq_slot, const int* cu_q, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    return oe_launch(token_shift_mix_kernel<float>, dim3(n_tokens), dim3(256), 0, st, out, h, mu, prev_state, n_mix, n_tokens,
                     D, tok_seq, seq_slot, cu_q);
}
int oe_token_shift_mix_bf16(bf16* out, const bf16* h, const float* mu, const float* prev_state, int n_mix, int n_tokens,
                            int D, const int* tok_seq, const int* seq_slot, const int* cu_q, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    return oe_launch(token_shift_mix_kernel<bf16>, dim3(n_tokens), dim3(256), 0, st, out, h, mu, prev_state, n_mix, n_tokens,
                     D, tok_seq, seq_slot, cu_q);
}

int oe_last_rows_to_state_f32(float* state, const float* h, int D, const int* seq_slot, const int* cu_q, int n_seqs,
                              cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    return oe_launch(last_rows_to_state_kernel<float>, dim3(n_seqs), dim3(256), 0, st, state, h, D, seq_slot, cu_q);
}
int oe_last_rows_to_state_bf16(float* state, const bf16* h, int D, const int* seq_slot, const int* cu_q, int n_seqs,
                               cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    return oe_launch(last_rows_to_state_kernel<bf16>, dim3(n_seqs), dim3(256), 0, st, state, h, D, seq_slot, cu_q);
}

int oe_decay_scan(float* o, float* state, const float* r, const float* k, const float* v, const float* z, long long stride,
                  const float* u, const float* w0, const int* seq_slot, const int* cu_q, int n_seqs, int H, int d,
                  cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (d < 1 || d > 256 || H < 1 || n_seqs > 65535) return OE_ERR_UNSUPPORTED;
    const int L = lanes_per_column(d, d), per = d / L;
    const dim3 grid(H, n_seqs), block(round_up_warp(d * L));
    if (block.x > (per > 32 ? 256u : 512u)) return OE_ERR_UNSUPPORTED;
#define OE_SCAN(PER, LL) \
    if (L == LL && per <= PER) return oe_launch(decay_scan_kernel<PER, LL>, grid, block, 0, st, o, state, r, k, v, z, stride, u, w0, seq_slot, cu_q, H, d);
    OE_SCAN(8, 8) OE_SCAN(16, 8) OE_SCAN(32, 8)
    OE_SCAN(8, 4) OE_SCAN(16, 4) OE_SCAN(32, 4) OE_SCAN(64, 4)
    OE_SCAN(8, 2) OE_SCAN(16, 2) OE_SCAN(32, 2) OE_SCAN(64, 2) OE_SCAN(128, 2)
    OE_SCAN(8, 1) OE_SCAN(16, 1) OE_SCAN(32, 1) OE_SCAN(64, 1) OE_SCAN(128, 1) OE_SCAN(256, 1)
#undef OE_SCAN
    return OE_ERR_UNSUPPORTED;
}

}  // extern "C"
