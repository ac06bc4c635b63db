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

constexpr int MAX_TAPS = 32;
constexpr int MAX_CHUNK = 16;       // tokens whose vectors are staged at once (fewer where they are long)

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// proj row: [q: G*dk | k: G*dk | v: H*dv | gate: H*dv | beta: H | a: H].  grid (tokens, 2 G + value chunks):
// block y < 2 G takes one q or k head (convolution, silu, unit vector), the others VCHUNK value channels each;
// block y == 0 also writes the token's decays and step sizes.
// out_qkv row [q | k | v] (C = 2 G dk + H dv), out_gb row [g: H | beta: H].
constexpr int VCHUNK = 256;
__device__ __forceinline__ float conv_silu(const float* proj, int P, const float* __restrict__ conv_w, int taps,
                                           const float* st, int C, int t, int rel, int c) {
    float acc = 0.f;
    for (int j = 0; j < taps; j++) {
        const int r = rel - (taps - 1) + j;
        const float x = r >= 0 ? proj[(size_t)(t - rel + r) * P + c] : st[(size_t)(rel + j) * C + c];
        acc = fmaf(conv_w[(size_t)c * taps + j], x, acc);
    }
    return silu_f(acc);
}

__global__ void __launch_bounds__(128)
short_conv_prepare_kernel(float* out_qkv, float* out_gb, const float* proj, int P,
                          const float* __restrict__ conv_w, int taps, const float* conv_state,
                          const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                          const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                          const int* __restrict__ cu_q, int G, int H, int dk, int dv, float q_scale) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, part = blockIdx.y;
    const int b = tok_seq[t];
    if (b < 0) return;
    const int slot = seq_slot[b];
    const int rel = t - cu_q[b];                // index of the token among its sequence's tokens of this step
    const int nqk = 2 * G * dk, C = nqk + H * dv;
    const float* st = conv_state + (size_t)slot * (taps - 1) * C;
    if (part < 2 * G) {
        // dk <= 256: a thread keeps its (up to two) channels in registers
        const int c0 = part * dk;
        float y[2] = {0.f, 0.f};
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int d = threadIdx.x + e * 128;
            if (d < dk) { y[e] = conv_silu(proj, P, conv_w, taps, st, C, t, rel, c0 + d); ss = fmaf(y[e], y[e], ss); }
        }
        ss = block_sum(ss, red);
        const float s = (1.f / sqrtf(ss + 1e-6f)) * (part < G ? q_scale : 1.f);
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int d = threadIdx.x + e * 128;
            if (d < dk) out_qkv[(size_t)t * C + c0 + d] = y[e] * s;
        }
    } else {
        const int c0 = nqk + (part - 2 * G) * VCHUNK;
        for (int c = c0 + threadIdx.x; c < min(c0 + VCHUNK, C); c += 128)
            out_qkv[(size_t)t * C + c] = conv_silu(proj, P, conv_w, taps, st, C, t, rel, c);
    }
    if (part == 0) {
        const float* row = proj + (size_t)t * P;
        for (int hh = threadIdx.x; hh < H; hh += blockDim.x) {
            const float bt = row[C + H * dv + hh], a = row[C + H * dv + H + hh];
            out_gb[(size_t)t * 2 * H + hh] = expf(-expf(A_log[hh]) * softplus_f(a + dt_bias[hh]));
            out_gb[(size_t)t * 2 * H + H + hh] = 1.f / (1.f + expf(-bt));
        }
    }
}

// grid (sequences, channel chunks); a thread owns whole channels, so it reads a channel's old rows before it
// writes them.
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
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= C) return;
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

// Sum over the L adjacent lanes that share a column (L a power of two up to 8), the same order everywhere.
template <int L>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = 1; o < L; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Which row of its column lane l keeps in register ii: with one lane the rows in order; with L lanes
// groups of four consecutive rows dealt round robin, so that the lanes of a column read consecutive 16-byte
// pieces of a staged vector.
template <int L>
__device__ __forceinline__ int lane_row(int ii, int l) { return L == 1 ? ii : ((ii >> 2) * 4 * L + 4 * l + (ii & 3)); }

// grid (H * column tiles, B).  A block owns `cols` columns of S[dk][dv] of one head of one sequence; column j
// belongs to L adjacent threads, thread l of them keeps dk / L rows in registers (lane_row).  The step's
// tokens are walked in order in chunks: while one chunk is computed, the next chunk's k, q (dk each), the
// block's v columns, the decay and the step size arrive in shared memory by asynchronous copies.
// qkv row [q: G*dk | k: G*dk | v: H*dv], gb row [g: H | beta: H]; o [T, H*dv] float32.
template <int PER, int L, int NC, bool EXACT>
__global__ void __launch_bounds__(PER >= 64 ? 256 : 512)
delta_rule_scan_kernel(float* o, float* state, const float* qkv, const float* gb,
                       const int* __restrict__ seq_slot, const int* __restrict__ cu_q,
                       int G, int H, int dk, int dv, int cols, int chunk) {
    extern __shared__ __align__(16) float stage_mem[];
    pdl_launch_dependents();
    pdl_wait();
    const int tiles = (dv + cols - 1) / cols;
    const int h = blockIdx.x / tiles, col0 = (blockIdx.x % tiles) * cols, b = blockIdx.y;
    // a thread keeps its rows of NC adjacent columns: what it reads of k and q serves all of them
    const int jj = (threadIdx.x / L) * NC, l = threadIdx.x % L, j = col0 + jj;
    const int slot = seq_slot[b];
    const int row0 = cu_q[b], n = cu_q[b + 1] - row0;
    if (slot < 0 || n <= 0) return;
    const int g = h / (H / G);
    const int C = 2 * G * dk + H * dv;
    // EXACT: every lane keeps exactly PER rows, known at compile time (with the count only known at run time
    // every unrolled instruction carries a predicate: a scan of 2,048 tokens then took 1.10 instead of 0.74 ms)
    const int per = EXACT ? PER : dk / L;
    bool mine[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) mine[c] = jj + c < cols && j + c < dv;
    const int tokf = (2 * dk + cols + 2 + 3) / 4 * 4;            // floats of a staged token: k, q, v columns, g, beta
    float* S = state + (((size_t)slot * H + h) * dk) * dv;
    float s[NC][PER];
#pragma unroll
    for (int c = 0; c < NC; c++)
#pragma unroll
        for (int i = 0; i < PER; i++) s[c][i] = (mine[c] && i < per) ? S[(size_t)lane_row<L>(i, l) * dv + j + c] : 0.f;

    // 16-byte copies where every piece starts on a 16-byte boundary, else 4-byte copies
    const bool vec = ((dk | cols | dv | C) & 3) == 0 && (((uintptr_t)qkv) & 15) == 0;
    auto issue = [&](int c0, float* dst) {
        const int cn = min(chunk, n - c0);
        if (vec) {
            const int kq4 = dk / 2, v4 = cols / 4, vpt = kq4 + v4;        // 16-byte pieces of a token: k and q, v columns
            auto piece = [&](int tt, int r) {
                const float* rowp = qkv + (size_t)(row0 + c0 + tt) * C;
                float* d = dst + tt * tokf;
                if (r < dk / 4) cp_async16(d + 4 * r, rowp + (size_t)(G + g) * dk + 4 * r);
                else if (r < kq4) cp_async16(d + 4 * r, rowp + (size_t)g * dk + 4 * (r - dk / 4));
                else if (col0 + 4 * (r - kq4) < dv) cp_async16(d + 4 * r, rowp + (size_t)2 * G * dk + (size_t)h * dv + col0 + 4 * (r - kq4));
            };
            // a power-of-two group of threads per token (shifts, no division): thread (tt, r) copies piece r
            const int lg = 32 - __clz(max(vpt - 1, 1)), span = 1 << lg;
            if (span <= (int)blockDim.x) {
                const int r = threadIdx.x & (span - 1);
                if (r < vpt)
                    for (int tt = threadIdx.x >> lg; tt < cn; tt += blockDim.x >> lg) piece(tt, r);
            } else {
                for (int tt = 0; tt < cn; tt++)
                    for (int r = threadIdx.x; r < vpt; r += blockDim.x) piece(tt, r);
            }
            for (int e = threadIdx.x; e < cn * 2; e += blockDim.x)
                cp_async4(dst + (e >> 1) * tokf + 2 * dk + cols + (e & 1), gb + (size_t)(row0 + c0 + (e >> 1)) * 2 * H + (size_t)(e & 1) * H + h);
            cp_async_commit();
            return;
        }
        for (int e = threadIdx.x; e < cn * tokf; e += blockDim.x) {
            const int tt = e / tokf, r = e % tokf;
            const size_t row = (size_t)(row0 + c0 + tt);
            const float* src = nullptr;
            if (r < dk) src = qkv + row * C + (size_t)(G + g) * dk + r;
            else if (r < 2 * dk) src = qkv + row * C + (size_t)g * dk + (r - dk);
            else if (r < 2 * dk + cols) { if (col0 + r - 2 * dk < dv) src = qkv + row * C + (size_t)2 * G * dk + (size_t)h * dv + col0 + (r - 2 * dk); }
            else if (r < 2 * dk + cols + 2) src = gb + row * 2 * H + (size_t)(r - 2 * dk - cols) * H + h;
            if (src) cp_async4(dst + e, src);
        }
        cp_async_commit();
    };
    const int stagef = chunk * tokf;
    issue(0, stage_mem);
    int buf = 0;
    for (int c0 = 0; c0 < n; c0 += chunk, buf ^= 1) {
        const int cn = min(chunk, n - c0);
        if (c0 + chunk < n) { issue(c0 + chunk, stage_mem + (buf ^ 1) * stagef); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        const float* base = stage_mem + buf * stagef;
        // The read-out o = S^T q of a token does not feed the next token's update, so its sum over the lanes
        // and its store are issued behind the next token's products with k (pend: the token it belongs to).
        float pend_acc[NC];
#pragma unroll
        for (int c = 0; c < NC; c++) pend_acc[c] = 0.f;
        long long pend = -1;
        for (int tt = 0; tt < cn; tt++) {
            const float* tk = base + tt * tokf;
            const float decay = tk[2 * dk + cols], beta = tk[2 * dk + cols + 1];
            float v[NC], d[NC][4];
#pragma unroll
            for (int c = 0; c < NC; c++) {
                v[c] = tk[2 * dk + (jj + c < cols ? jj + c : 0)];
                d[c][0] = d[c][1] = d[c][2] = d[c][3] = 0.f;
            }
            // k . (g S) = g (k . S): the products with k use the state as the last token left it, and the
            // state is scaled while their sum travels between the lanes
            if (L == 1) {
#pragma unroll
                for (int i = 0; i < PER; i++)
                    if (i < per) {
                        const float kv = tk[i];
#pragma unroll
                        for (int c = 0; c < NC; c++) d[c][0] = fmaf(kv, s[c][i], d[c][0]);
                    }
            } else {
                const float4* k4 = reinterpret_cast<const float4*>(tk);
#pragma unroll
                for (int i = 0; i < PER; i += 4) {
                    if (i < per) {
                        const float4 kv = k4[(i >> 2) * L + l];
#pragma unroll
                        for (int c = 0; c < NC; c++) {
                            d[c][0] = fmaf(kv.x, s[c][i], d[c][0]); d[c][1] = fmaf(kv.y, s[c][i + 1], d[c][1]);
                            d[c][2] = fmaf(kv.z, s[c][i + 2], d[c][2]); d[c][3] = fmaf(kv.w, s[c][i + 3], d[c][3]);
                        }
                    }
                }
            }
            float dsum[NC];
#pragma unroll
            for (int c = 0; c < NC; c++) dsum[c] = (d[c][0] + d[c][1]) + (d[c][2] + d[c][3]);
#pragma unroll
            for (int sh = 1; sh < L; sh <<= 1) {
                float other[NC];
#pragma unroll
                for (int c = 0; c < NC; c++) other[c] = __shfl_xor_sync(0xffffffffu, dsum[c], sh);
                if (sh == 1) {
#pragma unroll
                    for (int c = 0; c < NC; c++)
#pragma unroll
                        for (int i = 0; i < PER; i++)
                            if (i < per) s[c][i] *= decay;
                }
#pragma unroll
                for (int c = 0; c < NC; c++) dsum[c] += other[c];
            }
            if (L == 1) {
#pragma unroll
                for (int c = 0; c < NC; c++)
#pragma unroll
                    for (int i = 0; i < PER; i++)
                        if (i < per) s[c][i] *= decay;
            }
            if (pend >= 0) {
#pragma unroll
                for (int c = 0; c < NC; c++) {
                    const float acc = lanes_sum<L>(pend_acc[c]);
                    if (mine[c] && l == 0) o[(size_t)pend * (size_t)(H * dv) + (size_t)h * dv + j + c] = acc;
                }
            }
            float u[NC], a[NC][4];
#pragma unroll
            for (int c = 0; c < NC; c++) {
                u[c] = beta * (v[c] - decay * dsum[c]);
                a[c][0] = a[c][1] = a[c][2] = a[c][3] = 0.f;
            }
            if (L == 1) {
#pragma unroll
                for (int i = 0; i < PER; i++)
                    if (i < per) {
                        const float kv = tk[i], qv = tk[dk + i];
#pragma unroll
                        for (int c = 0; c < NC; c++) { s[c][i] = fmaf(kv, u[c], s[c][i]); a[c][0] = fmaf(qv, s[c][i], a[c][0]); }
                    }
            } else {
                const float4* k4 = reinterpret_cast<const float4*>(tk);
                const float4* q4 = reinterpret_cast<const float4*>(tk + dk);
#pragma unroll
                for (int i = 0; i < PER; i += 4) {
                    if (i < per) {
                        const float4 kv = k4[(i >> 2) * L + l], qv = q4[(i >> 2) * L + l];
#pragma unroll
                        for (int c = 0; c < NC; c++) {
                            s[c][i] = fmaf(kv.x, u[c], s[c][i]); s[c][i + 1] = fmaf(kv.y, u[c], s[c][i + 1]);
                            s[c][i + 2] = fmaf(kv.z, u[c], s[c][i + 2]); s[c][i + 3] = fmaf(kv.w, u[c], s[c][i + 3]);
                            a[c][0] = fmaf(qv.x, s[c][i], a[c][0]); a[c][1] = fmaf(qv.y, s[c][i + 1], a[c][1]);
                            a[c][2] = fmaf(qv.z, s[c][i + 2], a[c][2]); a[c][3] = fmaf(qv.w, s[c][i + 3], a[c][3]);
                        }
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < NC; c++) pend_acc[c] = (a[c][0] + a[c][1]) + (a[c][2] + a[c][3]);
            pend = (long long)(row0 + c0 + tt);
        }
        if (pend >= 0) {
#pragma unroll
            for (int c = 0; c < NC; c++) {
                const float acc = lanes_sum<L>(pend_acc[c]);
                if (mine[c] && l == 0) o[(size_t)pend * (size_t)(H * dv) + (size_t)h * dv + j + c] = acc;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < NC; c++) {
        if (mine[c]) {
#pragma unroll
            for (int i = 0; i < PER; i++)
                if (i < per) S[(size_t)lane_row<L>(i, l) * dv + j + c] = s[c][i];
        }
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

// grid (H * column tiles, B), columns and lanes as in the delta rule's scan.  Staged per token: r, k, the
// decay's argument z (turned into w = exp(-exp(z + w0)) once it has arrived), u * k, and the block's v columns.
// r, k, v, z: float32 rows of H*d with one row stride; u, w0: [H*d].
template <int PER, int L, bool EXACT>
__global__ void __launch_bounds__(PER >= 64 ? 256 : 512)
decay_scan_kernel(float* o, float* state, const float* r, const float* k, const float* v, const float* z,
                  long long stride, const float* __restrict__ u, const float* __restrict__ w0,
                  const int* __restrict__ seq_slot, const int* __restrict__ cu_q, int H, int d, int cols, int chunk) {
    extern __shared__ __align__(16) float stage_mem[];
    pdl_launch_dependents();
    pdl_wait();
    const int tiles = (d + cols - 1) / cols;
    const int h = blockIdx.x / tiles, col0 = (blockIdx.x % tiles) * cols, b = blockIdx.y;
    const int jj = threadIdx.x / L, l = threadIdx.x % L, j = col0 + jj;
    const int slot = seq_slot[b];
    const int row0 = cu_q[b], n = cu_q[b + 1] - row0;
    if (slot < 0 || n <= 0) return;
    const int per = EXACT ? PER : d / L;
    const bool mine = jj < cols && j < d;
    const int dp = (d + 3) / 4 * 4;
    const int tokf = 4 * dp + (cols + 3) / 4 * 4;                // r, k, z -> w, u * k, v columns
    float* S = state + (((size_t)slot * H + h) * d) * d;
    float s[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) s[i] = (mine && i < per) ? S[(size_t)lane_row<L>(i, l) * d + j] : 0.f;

    const bool vec = ((d | cols) & 3) == 0 && (stride & 3) == 0 &&
                     ((((uintptr_t)r) | ((uintptr_t)k) | ((uintptr_t)v) | ((uintptr_t)z)) & 15) == 0;
    auto issue = [&](int c0, float* dst) {
        const int cn = min(chunk, n - c0);
        if (vec) {
            const int d4 = d / 4, v4 = cols / 4, vpt = 3 * d4 + v4;      // 16-byte pieces of a token: r, k, z, v columns
            auto piece = [&](int tt, int q) {
                const size_t at = (size_t)(row0 + c0 + tt) * stride + (size_t)h * d;
                float* dd = dst + tt * tokf;
                if (q < d4) cp_async16(dd + 4 * q, r + at + 4 * q);
                else if (q < 2 * d4) cp_async16(dd + dp + 4 * (q - d4), k + at + 4 * (q - d4));
                else if (q < 3 * d4) cp_async16(dd + 2 * dp + 4 * (q - 2 * d4), z + at + 4 * (q - 2 * d4));
                else if (col0 + 4 * (q - 3 * d4) < d) cp_async16(dd + 4 * dp + 4 * (q - 3 * d4), v + at + col0 + 4 * (q - 3 * d4));
            };
            const int lg = 32 - __clz(max(vpt - 1, 1)), span = 1 << lg;
            if (span <= (int)blockDim.x) {
                const int q = threadIdx.x & (span - 1);
                if (q < vpt)
                    for (int tt = threadIdx.x >> lg; tt < cn; tt += blockDim.x >> lg) piece(tt, q);
            } else {
                for (int tt = 0; tt < cn; tt++)
                    for (int q = threadIdx.x; q < vpt; q += blockDim.x) piece(tt, q);
            }
            cp_async_commit();
            return;
        }
        for (int e = threadIdx.x; e < cn * tokf; e += blockDim.x) {
            const int tt = e / tokf, q = e % tokf, which = q / dp, i = q % dp;
            const size_t at = (size_t)(row0 + c0 + tt) * stride + (size_t)h * d;
            const float* src = nullptr;
            if (which < 3) { if (i < d) src = (which == 0 ? r : which == 1 ? k : z) + at + i; }
            else if (which == 4) { if (i < cols && col0 + i < d) src = v + at + col0 + i; }
            if (src) cp_async4(dst + e, src);
        }
        cp_async_commit();
    };
    const int stagef = chunk * tokf;
    issue(0, stage_mem);
    int buf = 0;
    for (int c0 = 0; c0 < n; c0 += chunk, buf ^= 1) {
        const int cn = min(chunk, n - c0);
        if (c0 + chunk < n) { issue(c0 + chunk, stage_mem + (buf ^ 1) * stagef); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        float* base = stage_mem + buf * stagef;
        for (int e = threadIdx.x; e < cn * d; e += blockDim.x) {
            const int tt = e / d, i = e % d;
            float* tk = base + tt * tokf;
            tk[2 * dp + i] = expf(-expf(tk[2 * dp + i] + w0[(size_t)h * d + i]));
            tk[3 * dp + i] = u[(size_t)h * d + i] * tk[dp + i];
        }
        __syncthreads();
        for (int tt = 0; tt < cn; tt++) {
            const float* tk = base + tt * tokf;
            const float vj = tk[4 * dp + (jj < cols ? jj : 0)];
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            if (L == 1) {
#pragma unroll
                for (int i = 0; i < PER; i++) {
                    if (i < per) {
                        a0 = fmaf(tk[i], fmaf(tk[3 * dp + i], vj, s[i]), a0);
                        s[i] = fmaf(tk[2 * dp + i], s[i], tk[dp + i] * vj);
                    }
                }
            } else {
                const float4* r4 = reinterpret_cast<const float4*>(tk);
                const float4* k4 = reinterpret_cast<const float4*>(tk + dp);
                const float4* w4 = reinterpret_cast<const float4*>(tk + 2 * dp);
                const float4* uk4 = reinterpret_cast<const float4*>(tk + 3 * dp);
#pragma unroll
                for (int i = 0; i < PER; i += 4) {
                    if (i < per) {
                        const int at = (i >> 2) * L + l;
                        const float4 rv = r4[at], kv = k4[at], wv = w4[at], uv = uk4[at];
                        a0 = fmaf(rv.x, fmaf(uv.x, vj, s[i]), a0); a1 = fmaf(rv.y, fmaf(uv.y, vj, s[i + 1]), a1);
                        a2 = fmaf(rv.z, fmaf(uv.z, vj, s[i + 2]), a2); a3 = fmaf(rv.w, fmaf(uv.w, vj, s[i + 3]), a3);
                        s[i] = fmaf(wv.x, s[i], kv.x * vj); s[i + 1] = fmaf(wv.y, s[i + 1], kv.y * vj);
                        s[i + 2] = fmaf(wv.z, s[i + 2], kv.z * vj); s[i + 3] = fmaf(wv.w, s[i + 3], kv.w * vj);
                    }
                }
            }
            const float acc = lanes_sum<L>((a0 + a1) + (a2 + a3));
            if (mine && l == 0) o[(size_t)(row0 + c0 + tt) * (size_t)(H * d) + (size_t)h * d + j] = acc;
        }
        __syncthreads();
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < PER; i++)
            if (i < per) S[(size_t)lane_row<L>(i, l) * d + j] = s[i];
    }
}

// How a scan is laid out: lanes per column (the most of 8, 4, 2 that leave each lane a multiple of four rows
// and at least eight, else 1), columns per block (up to 32), tokens per staged chunk (the most of 16, 8, 4, 2, 1
// whose two stages fit 48 KB).  Measured on a B200, one sequence of 2,048 tokens, 16 heads of 128 x 128
// (us; lanes x columns): 8 x 32 1,116, 8 x 16 1,138, 4 x 32 2,088, 2 x 32 2,586; 16 lanes: 833 but a decode
// step of 64 sequences 87 instead of 53 (a lane's share of a column's rows is what the time follows: the
// kernel issues about 190 instructions a token and warp, with one or two warps a scheduler).
struct ScanPlan { int L, cols, threads, chunk; size_t smem; };
inline ScanPlan scan_plan(int rows, int ncols, int tok_floats_without_cols, int pad_cols) {
    ScanPlan p;
    p.L = 1;
    for (int L = 8; L > 1; L >>= 1)
        if (rows % (4 * L) == 0 && rows / L >= 8) { p.L = L; break; }
    p.cols = ncols < 32 ? ncols : 32;
    while (p.cols * p.L > (rows / p.L > 32 ? 256 : 512)) p.cols /= 2;
    p.threads = (p.cols * p.L + 31) / 32 * 32;
    const int tokf = pad_cols ? tok_floats_without_cols + (p.cols + 3) / 4 * 4 : (tok_floats_without_cols + p.cols + 3) / 4 * 4;
    p.chunk = MAX_CHUNK;
    while (p.chunk > 1 && (size_t)2 * p.chunk * tokf * sizeof(float) > 48 * 1024) p.chunk /= 2;
    p.smem = (size_t)2 * p.chunk * tokf * sizeof(float);
    return p;
}

}  // namespace

extern "C" {

int oe_short_conv_prepare(float* out_qkv, float* out_gb, const float* proj, int P, const float* conv_w, int taps,
                          const float* conv_state, const float* A_log, const float* dt_bias, const int* tok_seq,
                          const int* seq_slot, const int* cu_q, int n_tokens, int G, int H, int dk, int dv, float q_scale,
                          cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (taps < 1 || taps > MAX_TAPS || G < 1 || H % G) return OE_ERR_UNSUPPORTED;
    if (dk > 256) return OE_ERR_UNSUPPORTED;
    const int parts = 2 * G + (H * dv + VCHUNK - 1) / VCHUNK;
    if (parts > 65535) return OE_ERR_UNSUPPORTED;
    return oe_launch(short_conv_prepare_kernel, dim3(n_tokens, parts), dim3(128), 0, st, out_qkv, out_gb, proj, P, conv_w, taps,
                     conv_state, A_log, dt_bias, tok_seq, seq_slot, cu_q, G, H, dk, dv, q_scale);
}

int oe_conv_state_update(float* conv_state, const float* proj, int P, int C, int taps, const int* seq_slot,
                         const int* cu_q, int n_seqs, cudaStream_t st) {
    if (n_seqs <= 0 || taps <= 1) return 0;
    if (taps > MAX_TAPS) return OE_ERR_UNSUPPORTED;
    return oe_launch(conv_state_update_kernel, dim3(n_seqs, (C + 255) / 256), dim3(256), 0, st, conv_state, proj, P, C, taps, seq_slot, cu_q);
}

int oe_delta_rule_scan(float* o, float* state, const float* qkv, const float* gb, const int* seq_slot, const int* cu_q,
                       int n_seqs, int G, int H, int dk, int dv, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || dv > 4096 || G < 1 || H % G || n_seqs > 65535) return OE_ERR_UNSUPPORTED;
    const ScanPlan p = scan_plan(dk, dv, 2 * dk + 2, 0);
    if (p.cols < 1 || p.smem > 48 * 1024) return OE_ERR_UNSUPPORTED;
    const int L = p.L, per = dk / L;
    // Two columns a thread where a lane keeps at most 16 rows of each (registers) and the columns pair up: what a
    // thread reads of k and q then serves both (16 heads of 128 x 128, us, one / two columns: 8 sequences of 512
    // tokens 733 / 449, 64 sequences of one token 52 / 46, one sequence of 2,048 tokens 1,364 / 1,102).
    const int nc = (per <= 16 && p.cols % 2 == 0 && L > 1) ? 2 : 1;
    const dim3 grid(H * ((dv + p.cols - 1) / p.cols), n_seqs), block(((p.cols / nc) * L + 31) / 32 * 32);
#define OE_SCAN(PER, LL) \
    if (L == LL && per <= PER) { \
        if (nc == 2 && PER <= 16) { \
            if (per == PER) return oe_launch(delta_rule_scan_kernel<(PER <= 16 ? PER : 16), LL, 2, true>, grid, block, p.smem, st, o, state, qkv, gb, seq_slot, cu_q, G, H, dk, dv, p.cols, p.chunk); \
            return oe_launch(delta_rule_scan_kernel<(PER <= 16 ? PER : 16), LL, 2, false>, grid, block, p.smem, st, o, state, qkv, gb, seq_slot, cu_q, G, H, dk, dv, p.cols, p.chunk); \
        } \
        if (per == PER) return oe_launch(delta_rule_scan_kernel<PER, LL, 1, true>, grid, block, p.smem, st, o, state, qkv, gb, seq_slot, cu_q, G, H, dk, dv, p.cols, p.chunk); \
        return oe_launch(delta_rule_scan_kernel<PER, LL, 1, false>, grid, block, p.smem, st, o, state, qkv, gb, seq_slot, cu_q, G, H, dk, dv, p.cols, p.chunk); \
    }
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
    const ScanPlan p = scan_plan(d, d, 4 * ((d + 3) / 4 * 4), 1);
    if (p.cols < 1 || p.smem > 48 * 1024) return OE_ERR_UNSUPPORTED;
    const int L = p.L, per = d / L;
    const dim3 grid(H * ((d + p.cols - 1) / p.cols), n_seqs), block(p.threads);
#define OE_SCAN(PER, LL) \
    if (L == LL && per <= PER) { \
        if (per == PER) return oe_launch(decay_scan_kernel<PER, LL, true>, grid, block, p.smem, st, o, state, r, k, v, z, stride, u, w0, seq_slot, cu_q, H, d, p.cols, p.chunk); \
        return oe_launch(decay_scan_kernel<PER, LL, false>, grid, block, p.smem, st, o, state, r, k, v, z, stride, u, w0, seq_slot, cu_q, H, d, p.cols, p.chunk); \
    }
    OE_SCAN(8, 8) OE_SCAN(16, 8) OE_SCAN(32, 8)
    OE_SCAN(8, 4) OE_SCAN(16, 4) OE_SCAN(32, 4) OE_SCAN(64, 4)
    OE_SCAN(8, 2) OE_SCAN(16, 2) OE_SCAN(32, 2) OE_SCAN(64, 2) OE_SCAN(128, 2)
    OE_SCAN(8, 1) OE_SCAN(16, 1) OE_SCAN(32, 1) OE_SCAN(64, 1) OE_SCAN(128, 1) OE_SCAN(256, 1)
#undef OE_SCAN
    return OE_ERR_UNSUPPORTED;
}

}  // extern "C"
