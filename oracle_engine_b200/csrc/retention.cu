// Retention: linear attention with one fixed decay per head and no softmax or denominator.
//
// Per sequence and head, over the step's tokens in order, with S [dk, dv] the sequence's state (float32):
//     S <- gamma_h S + k_t v_t^T        o_t = S^T q_t
// q_t and k_t are the projections turned by the token's position (the first `rot` dimensions of a head,
// dimension i < rot/2 paired with i + rot/2, cosine and sine from a float32 table [positions, rot/2]) and
// k_t is multiplied by k_scale after the turn; all of that in float32, while the tokens are staged.
//
// Two kernels compute it; the host picks by the longest run of tokens a sequence brings in the step.
//
// retention_chunks (prompts and pieces of prompts): a block owns 16 columns of one (sequence, head) and walks the
// sequence's tokens in chunks of 32.  With S the state before a chunk whose tokens are 0 .. n-1:
//     A_tj = gamma^(t-j) q_t . k_j  (j <= t)        o_t = sum_j A_tj v_j + gamma^(t+1) S^T q_t
//     S   <- gamma^n S + sum_j gamma^(n-1-j) k_j v_j^T
// which are the same sums as the recurrence, taken chunk by chunk: the products of a chunk do not wait for one
// another, only the state goes from chunk to chunk.  The powers of gamma are rounded from double precision.
//
// retention_scan (single tokens and very short pieces): a block owns up to `cols` columns of one (sequence, head); L lanes share a column, lane l
// keeps rows l, l + L, ... of it in registers.  Tokens are staged in chunks into shared memory (q, k turned
// and scaled, and the block's slice of v); per token a lane updates its rows, multiplies them with q and the
// L partial sums are added by shuffles.  Prompts, pieces of prompts and single tokens run the same code and
// the same order of operations, so the state after a token does not depend on how the tokens were cut.
#include "common.cuh"

namespace {

constexpr int CHUNK = 16;

template <int L> __device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int PER, int L>
__global__ void __launch_bounds__(256)
retention_scan_kernel(float* o, float* state, const float* proj, long long stride, int off_q, int off_k, int off_v,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot, float k_scale,
                      const float* __restrict__ decay, const int* __restrict__ seq_slot, const int* __restrict__ cu_q,
                      const int* __restrict__ tok_pos, int H, int dk, int dv, int cols) {
    extern __shared__ __align__(16) float stage[];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int slot = seq_slot[b];
    const int row0 = cu_q[b], n = cu_q[b + 1] - row0;
    if (slot < 0 || n <= 0) return;
    const int tiles = (dv + cols - 1) / cols;
    const int h = blockIdx.x / tiles, col0 = (blockIdx.x % tiles) * cols;
    const int l = threadIdx.x % L, c = threadIdx.x / L;
    const int col = col0 + c;
    const bool mine = c < cols && col < dv;
    const float gamma = decay[h];
    const int half = rot / 2;
    const int tokf = 2 * dk + cols;
    float* S = state + ((size_t)slot * H + h) * (size_t)dk * dv;

    float s[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int r = i * L + l;
        s[i] = (mine && r < dk) ? S[(size_t)r * dv + col] : 0.f;
    }
    for (int c0 = 0; c0 < n; c0 += CHUNK) {
        const int cn = n - c0 < CHUNK ? n - c0 : CHUNK;
        for (int e = threadIdx.x; e < cn * dk; e += blockDim.x) {
            const int tt = e / dk, i = e % dk;
            if (i >= half && i < rot) continue;
            const int t = row0 + c0 + tt;
            const float* pr = proj + (size_t)t * stride + (size_t)h * dk;
            float* tk = stage + tt * tokf;
            if (i < half) {
                const int pos = tok_pos[t];
                const float cs = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
                const float qu = pr[off_q + i], qv = pr[off_q + i + half];
                const float ku = pr[off_k + i], kv = pr[off_k + i + half];
                tk[i] = qu * cs - qv * sn;
                tk[i + half] = qv * cs + qu * sn;
                tk[dk + i] = (ku * cs - kv * sn) * k_scale;
                tk[dk + i + half] = (kv * cs + ku * sn) * k_scale;
            } else {
                tk[i] = pr[off_q + i];
                tk[dk + i] = pr[off_k + i] * k_scale;
            }
        }
        for (int e = threadIdx.x; e < cn * cols; e += blockDim.x) {
            const int tt = e / cols, j = e % cols;
            const int t = row0 + c0 + tt;
            stage[tt * tokf + 2 * dk + j] = (col0 + j < dv) ? proj[(size_t)t * stride + off_v + (size_t)h * dv + col0 + j] : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < cn; tt++) {
            const float* tk = stage + tt * tokf;
            const float vj = tk[2 * dk + (c < cols ? c : 0)];
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int i = 0; i < PER; i += 2) {
                const int r0 = i * L + l, r1 = (i + 1) * L + l;
                if (r0 < dk) {
                    s[i] = fmaf(gamma, s[i], tk[dk + r0] * vj);
                    a0 = fmaf(s[i], tk[r0], a0);
                }
                if (r1 < dk) {
                    s[i + 1] = fmaf(gamma, s[i + 1], tk[dk + r1] * vj);
                    a1 = fmaf(s[i + 1], tk[r1], a1);
                }
            }
            const float acc = lanes_sum<L>(a0 + a1);
            if (mine && l == 0) o[(size_t)(row0 + c0 + tt) * (size_t)(H * dv) + (size_t)h * dv + col] = acc;
        }
        __syncthreads();
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int r = i * L + l;
            if (r < dk) S[(size_t)r * dv + col] = s[i];
        }
    }
}


constexpr int CC = 32;          // tokens per chunk
constexpr int CT = 16;          // state columns per block
constexpr int CTHREADS = 128;

// R8: rows of a state column a thread keeps (dk <= 8 * R8).
template <int R8>
__global__ void __launch_bounds__(CTHREADS)
retention_chunk_kernel(float* o, float* state, const float* proj, long long stride, int off_q, int off_k, int off_v,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot, float k_scale,
                       const float* __restrict__ decay, const int* __restrict__ seq_slot, const int* __restrict__ cu_q,
                       const int* __restrict__ tok_pos, int H, int dk, int dv) {
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int slot = seq_slot[b];
    const int row0 = cu_q[b], n = cu_q[b + 1] - row0;
    if (slot < 0 || n <= 0) return;
    const int tiles = (dv + CT - 1) / CT;
    const int h = blockIdx.x / tiles, col0 = (blockIdx.x % tiles) * CT;
    const int tid = threadIdx.x;
    const int ld = dk + 1;                               // odd row stride: the dot products' reads spread over the banks
    float* Qs = sm;                                      // [CC][ld]
    float* Ks = Qs + CC * ld;                            // [CC][ld]
    float* Vs = Ks + CC * ld;                            // [CC][CT]
    float* As = Vs + CC * CT;                            // [CC][CC + 1]
    float* Ss = As + CC * (CC + 1);                      // [dk][CT]
    float* pw = Ss + (size_t)dk * CT;                    // [CC + 1]: gamma^0 .. gamma^CC
    const double gamma = (double)decay[h];
    if (tid <= CC) pw[tid] = (float)pow(gamma, (double)tid);
    const int half = rot / 2;
    float* S = state + ((size_t)slot * H + h) * (size_t)dk * dv;
    const int col = tid % CT, rg = tid / CT;             // this thread's state column and its rows rg, rg + 8, ...
    const bool mine = col0 + col < dv;
    float s[R8];
#pragma unroll
    for (int i = 0; i < R8; i++) {
        const int r = rg + 8 * i;
        s[i] = (mine && r < dk) ? S[(size_t)r * dv + col0 + col] : 0.f;
        if (r < dk) Ss[r * CT + col] = s[i];
    }
    for (int c0 = 0; c0 < n; c0 += CC) {
        const int cn = n - c0 < CC ? n - c0 : CC;
        // stage q and k (turned, k scaled) and this block's columns of v; rows past the chunk's tokens are zero
        for (int e = tid; e < CC * dk; e += CTHREADS) {
            const int tt = e / dk, i = e % dk;
            if (i >= half && i < rot) continue;
            float* qd = Qs + tt * ld;
            float* kd = Ks + tt * ld;
            if (tt >= cn) {
                qd[i] = 0.f; kd[i] = 0.f;
                if (i < half) { qd[i + half] = 0.f; kd[i + half] = 0.f; }
                continue;
            }
            const int t = row0 + c0 + tt;
            const float* pr = proj + (size_t)t * stride + (size_t)h * dk;
            if (i < half) {
                const int pos = tok_pos[t];
                const float cs = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
                const float qu = pr[off_q + i], qv = pr[off_q + i + half];
                const float ku = pr[off_k + i], kv = pr[off_k + i + half];
                qd[i] = qu * cs - qv * sn;
                qd[i + half] = qv * cs + qu * sn;
                kd[i] = (ku * cs - kv * sn) * k_scale;
                kd[i + half] = (kv * cs + ku * sn) * k_scale;
            } else {
                qd[i] = pr[off_q + i];
                kd[i] = pr[off_k + i] * k_scale;
            }
        }
        for (int e = tid; e < CC * CT; e += CTHREADS) {
            const int tt = e / CT, j = e % CT;
            Vs[e] = (tt < cn && col0 + j < dv)
                        ? proj[(size_t)(row0 + c0 + tt) * stride + off_v + (size_t)h * dv + col0 + j] : 0.f;
        }
        __syncthreads();
        // A: a thread computes a 2 x 4 piece (rows 2 ti, 2 ti + 1; columns 4 tj .. 4 tj + 3) if it touches j <= t
        {
            const int ti = tid / 8, tj = tid % 8;
            const int ta = 2 * ti, ja = 4 * tj;
            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            if (ja <= ta + 1) {
                const float* q0 = Qs + ta * ld;
                const float* kk = Ks + ja * ld;
                for (int r = 0; r < dk; r++) {
                    const float qa = q0[r], qb = q0[ld + r];
                    const float k0 = kk[r], k1 = kk[ld + r], k2 = kk[2 * ld + r], k3 = kk[3 * ld + r];
                    acc[0][0] = fmaf(qa, k0, acc[0][0]); acc[0][1] = fmaf(qa, k1, acc[0][1]);
                    acc[0][2] = fmaf(qa, k2, acc[0][2]); acc[0][3] = fmaf(qa, k3, acc[0][3]);
                    acc[1][0] = fmaf(qb, k0, acc[1][0]); acc[1][1] = fmaf(qb, k1, acc[1][1]);
                    acc[1][2] = fmaf(qb, k2, acc[1][2]); acc[1][3] = fmaf(qb, k3, acc[1][3]);
                }
            }
#pragma unroll
            for (int a = 0; a < 2; a++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int t = ta + a, j = ja + c;
                    As[t * (CC + 1) + j] = j <= t ? acc[a][c] * pw[t - j] : 0.f;
                }
        }
        __syncthreads();
        // o: thread (col, rg) takes the tokens rg, rg + 8, rg + 16, rg + 24
        {
            float inter[4] = {0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < dk; r++) {
                const float sv = Ss[r * CT + col];
#pragma unroll
                for (int i = 0; i < 4; i++) inter[i] = fmaf(Qs[(rg + 8 * i) * ld + r], sv, inter[i]);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int t = rg + 8 * i;
                if (t >= cn) continue;
                float acc = 0.f;
                for (int j = 0; j <= t; j++) acc = fmaf(As[t * (CC + 1) + j], Vs[j * CT + col], acc);
                acc = fmaf(pw[t + 1], inter[i], acc);
                if (mine) o[(size_t)(row0 + c0 + t) * (size_t)(H * dv) + (size_t)h * dv + col0 + col] = acc;
            }
        }
        __syncthreads();
        // S <- gamma^cn S + sum_j gamma^(cn-1-j) k_j v_j^T
        {
            const float g = pw[cn];
#pragma unroll
            for (int i = 0; i < R8; i++) s[i] *= g;
            for (int j = 0; j < cn; j++) {
                const float wv = pw[cn - 1 - j] * Vs[j * CT + col];
                const float* kr = Ks + j * ld + rg;
#pragma unroll
                for (int i = 0; i < R8; i++)
                    if (rg + 8 * i < dk) s[i] = fmaf(kr[8 * i], wv, s[i]);
            }
#pragma unroll
            for (int i = 0; i < R8; i++)
                if (rg + 8 * i < dk) Ss[(rg + 8 * i) * CT + col] = s[i];
        }
        __syncthreads();
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < R8; i++) {
            const int r = rg + 8 * i;
            if (r < dk) S[(size_t)r * dv + col0 + col] = s[i];
        }
    }
}

template <int R8>
int launch_chunks(dim3 grid, size_t smem, cudaStream_t st, float* o, float* state, const float* proj, long long stride,
                  int off_q, int off_k, int off_v, const float* cos_t, const float* sin_t, int rot, float k_scale,
                  const float* decay, const int* seq_slot, const int* cu_q, const int* tok_pos, int H, int dk, int dv) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(retention_chunk_kernel<R8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    return oe_launch(retention_chunk_kernel<R8>, grid, dim3(CTHREADS), smem, st, o, state, proj, stride, off_q, off_k, off_v,
                     cos_t, sin_t, rot, k_scale, decay, seq_slot, cu_q, tok_pos, H, dk, dv);
}

}  // namespace

extern "C" {

int oe_retention_chunks(float* o, float* state, const float* proj, long long stride, int off_q, int off_k, int off_v,
                        const float* cos_t, const float* sin_t, int rot, float k_scale, const float* decay,
                        const int* seq_slot, const int* cu_q, const int* tok_pos, int n_seqs, int H, int dk, int dv,
                        cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || H < 1 || n_seqs > 65535 || rot < 0 || rot % 2 || rot > dk) return OE_ERR_UNSUPPORTED;
    const dim3 grid(H * ((dv + CT - 1) / CT), n_seqs);
    const size_t smem = sizeof(float) * ((size_t)2 * CC * (dk + 1) + CC * CT + CC * (CC + 1) + (size_t)dk * CT + CC + 1);
#define OE_RC(R8) \
    if (dk <= 8 * R8) return launch_chunks<R8>(grid, smem, st, o, state, proj, stride, off_q, off_k, off_v, cos_t, sin_t, rot, \
                                               k_scale, decay, seq_slot, cu_q, tok_pos, H, dk, dv);
    OE_RC(2) OE_RC(4) OE_RC(8) OE_RC(16) OE_RC(32)
#undef OE_RC
    return OE_ERR_UNSUPPORTED;
}

int oe_retention_scan(float* o, float* state, const float* proj, long long stride, int off_q, int off_k, int off_v,
                      const float* cos_t, const float* sin_t, int rot, float k_scale, const float* decay,
                      const int* seq_slot, const int* cu_q, const int* tok_pos, int n_seqs, int H, int dk, int dv,
                      cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || H < 1 || n_seqs > 65535 || rot < 0 || rot % 2 || rot > dk) return OE_ERR_UNSUPPORTED;
    const int L = dk <= 128 ? 4 : 8;
    const int per = (dk + L - 1) / L;
    // columns per block: 32, or 16 while the blocks of 32 would leave most SMs without one
    int cols = dv < 32 ? dv : 32;
    if (cols == 32 && (long long)n_seqs * H * ((dv + 31) / 32) < 148) cols = 16;
    const int tiles = (dv + cols - 1) / cols;
    const dim3 grid(H * tiles, n_seqs), block((cols * L + 31) / 32 * 32);
    const size_t smem = (size_t)CHUNK * (2 * dk + cols) * sizeof(float);
#define OE_RET(PER, LL) \
    if (L == LL && per <= PER) \
        return oe_launch(retention_scan_kernel<PER, LL>, grid, block, smem, st, o, state, proj, stride, off_q, off_k, off_v, \
                         cos_t, sin_t, rot, k_scale, decay, seq_slot, cu_q, tok_pos, H, dk, dv, cols);
    OE_RET(2, 4) OE_RET(4, 4) OE_RET(8, 4) OE_RET(16, 4) OE_RET(32, 4) OE_RET(32, 8)
#undef OE_RET
    return OE_ERR_UNSUPPORTED;
}

}  // extern "C"
