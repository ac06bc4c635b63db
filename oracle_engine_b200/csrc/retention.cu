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
// retention_chunks (prompts and pieces of prompts): every sequence's tokens of the step are cut into chunks of 32.
// With S the state before a chunk whose tokens are 0 .. n-1:
//     A_tj = gamma^(t-j) q_t . k_j  (j <= t)        o_t = sum_j A_tj v_j + gamma^(t+1) S^T q_t
//     S   <- gamma^n S + sum_j gamma^(n-1-j) k_j v_j^T
// which are the same sums as the recurrence, taken chunk by chunk.  Four launches: q and k turned in place; what
// every chunk adds to the state, all chunks and heads at once; the state carried from chunk to chunk, element by
// element (the only chain, one multiply-add per chunk); every chunk's outputs from the state before it, all chunks
// and heads at once.  The powers of gamma are rounded from double precision.  Scratch: a state per chunk and head.
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

// Which sequence and which of its chunks the g-th chunk of a step is (sequences in order, each cut into chunks
// of CC tokens from its first token of the step).  False if the step has fewer chunks.
__device__ __forceinline__ bool find_chunk(const int* __restrict__ cu_q, int n_seqs, int g, int& b, int& row, int& cn) {
    for (b = 0; b < n_seqs; b++) {
        const int len = cu_q[b + 1] - cu_q[b];
        const int nc = (len + CC - 1) / CC;
        if (g < nc) {
            row = cu_q[b] + g * CC;
            cn = len - g * CC < CC ? len - g * CC : CC;
            return true;
        }
        g -= nc;
    }
    return false;
}

// q and k of every token turned by its position and k scaled, in place in the projection rows.
__global__ void __launch_bounds__(128)
retention_prepare_kernel(float* proj, long long stride, int off_q, int off_k, const float* __restrict__ cos_t,
                         const float* __restrict__ sin_t, int rot, float k_scale, const int* __restrict__ tok_seq,
                         const int* __restrict__ tok_pos, int H, int dk) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (tok_seq[t] < 0) return;
    const int pos = tok_pos[t], half = rot / 2;
    float* pr = proj + (size_t)t * stride;
    for (int e = threadIdx.x; e < H * dk; e += blockDim.x) {
        const int i = e % dk;
        if (i >= half && i < rot) continue;
        float* q = pr + off_q + e;
        float* k = pr + off_k + e;
        if (i < half) {
            const float cs = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
            const float qu = q[0], qv = q[half], ku = k[0], kv = k[half];
            q[0] = qu * cs - qv * sn;
            q[half] = qv * cs + qu * sn;
            k[0] = (ku * cs - kv * sn) * k_scale;
            k[half] = (kv * cs + ku * sn) * k_scale;
        } else {
            k[0] *= k_scale;
        }
    }
}

// What a chunk adds to the state: W[g][h] = sum_j gamma^(n-1-j) k_j v_j^T  ([dk, dv]), one block per (chunk, head).
// 256 threads as 16 x 16: thread (ty, tx) owns rows ty + 16 i and columns tx + 16 c of a 64 x 128 piece.
__global__ void __launch_bounds__(256)
retention_chunk_state_kernel(float* W, const float* proj, long long stride, int off_k, int off_v,
                             const float* __restrict__ decay, const int* __restrict__ cu_q, int n_seqs, int H, int dk,
                             int dv) {
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    int b, row, cn;
    if (!find_chunk(cu_q, n_seqs, blockIdx.x, b, row, cn)) return;
    const int h = blockIdx.y, tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
    float* Ks = sm;                  // [CC][dk], row j times gamma^(cn-1-j)
    float* Vs = Ks + CC * dk;        // [CC][dv]
    __shared__ float pw[CC];
    const double gamma = (double)decay[h];
    if (tid < CC) pw[tid] = (float)pow(gamma, (double)tid);
    __syncthreads();
    for (int e = tid; e < CC * dk; e += 256) {
        const int j = e / dk, i = e % dk;
        Ks[e] = j < cn ? proj[(size_t)(row + j) * stride + off_k + (size_t)h * dk + i] * pw[cn - 1 - j] : 0.f;
    }
    for (int e = tid; e < CC * dv; e += 256) {
        const int j = e / dv, i = e % dv;
        Vs[e] = j < cn ? proj[(size_t)(row + j) * stride + off_v + (size_t)h * dv + i] : 0.f;
    }
    __syncthreads();
    float* Wg = W + ((size_t)blockIdx.x * H + h) * (size_t)dk * dv;
    for (int rb = 0; rb < dk; rb += 64) {
        for (int cb = 0; cb < dv; cb += 128) {
            float acc[4][8];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int c = 0; c < 8; c++) acc[i][c] = 0.f;
            for (int j = 0; j < cn; j++) {
                float kv[4], vv[8];
#pragma unroll
                for (int i = 0; i < 4; i++) { const int r = rb + ty + 16 * i; kv[i] = r < dk ? Ks[j * dk + r] : 0.f; }
#pragma unroll
                for (int c = 0; c < 8; c++) { const int col = cb + tx + 16 * c; vv[c] = col < dv ? Vs[j * dv + col] : 0.f; }
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int c = 0; c < 8; c++) acc[i][c] = fmaf(kv[i], vv[c], acc[i][c]);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int r = rb + ty + 16 * i;
                if (r >= dk) continue;
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    const int col = cb + tx + 16 * c;
                    if (col < dv) Wg[(size_t)r * dv + col] = acc[i][c];
                }
            }
        }
    }
}

// The state from chunk to chunk: for every element of a (sequence, head)'s state, S_before(chunk) is left in W in
// place of what the chunk adds, S <- gamma^n S + W, and the last S goes back to the sequence's state.
__global__ void __launch_bounds__(256)
retention_chunk_carry_kernel(float* W, float* state, const float* __restrict__ decay, const int* __restrict__ seq_slot,
                             const int* __restrict__ cu_q, int H, int dk, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.z, h = blockIdx.y;
    const int slot = seq_slot[b];
    const int len = cu_q[b + 1] - cu_q[b];
    if (slot < 0 || len <= 0) return;
    const int e = blockIdx.x * 256 + threadIdx.x;
    if (e >= dk * dv) return;
    int base = 0;
    for (int bb = 0; bb < b; bb++) base += (cu_q[bb + 1] - cu_q[bb] + CC - 1) / CC;
    const int nc = (len + CC - 1) / CC;
    const double gamma = (double)decay[h];
    const float g_full = (float)pow(gamma, (double)CC);
    const float g_last = (float)pow(gamma, (double)(len - (nc - 1) * CC));
    float* S = state + ((size_t)slot * H + h) * (size_t)dk * dv + e;
    float* w = W + ((size_t)base * H + h) * (size_t)dk * dv + e;
    const size_t step = (size_t)H * dk * dv;
    float s = *S;
    int c = 0;
    for (; c + 4 <= nc; c += 4) {                       // what the chunks add does not depend on the chain: four loads at once
        const float d0 = w[0], d1 = w[step], d2 = w[2 * step], d3 = w[3 * step];
        w[0] = s;        s = fmaf(g_full, s, d0);
        w[step] = s;     s = fmaf(g_full, s, d1);
        w[2 * step] = s; s = fmaf(g_full, s, d2);
        w[3 * step] = s; s = fmaf(c + 4 == nc ? g_last : g_full, s, d3);
        w += 4 * step;
    }
    for (; c < nc; c++) {
        const float d = w[0];
        w[0] = s;
        s = fmaf(c + 1 == nc ? g_last : g_full, s, d);
        w += step;
    }
    *S = s;
}

// A chunk's outputs: o_t = sum_{j <= t} gamma^(t-j) (q_t . k_j) v_j + gamma^(t+1) S_before^T q_t; one block per
// (chunk, head), 256 threads as 16 x 16: thread (ty, tx) owns tokens 2 ty, 2 ty + 1 and columns tx + 16 c.
__global__ void __launch_bounds__(256)
retention_chunk_out_kernel(float* o, const float* W, const float* proj, long long stride, int off_q, int off_k, int off_v,
                           const float* __restrict__ decay, const int* __restrict__ cu_q, int n_seqs, int H, int dk,
                           int dv) {
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    int b, row, cn;
    if (!find_chunk(cu_q, n_seqs, blockIdx.x, b, row, cn)) return;
    const int h = blockIdx.y, tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
    const int ld = dk + 1;
    float* Qs = sm;                          // [CC][ld]
    float* Ks = Qs + CC * ld;                // [CC][ld]
    float* As = Ks + CC * ld;                // [CC][CC + 1]
    float* Vs = As + CC * (CC + 1);          // [CC][128]: a block of columns of v
    float* Sb = Vs + CC * 128;               // [32][128]: a block of rows and columns of S_before
    float* pw = Sb + 32 * 128;               // [CC + 1]
    const double gamma = (double)decay[h];
    if (tid <= CC) pw[tid] = (float)pow(gamma, (double)tid);
    for (int e = tid; e < CC * dk; e += 256) {
        const int j = e / dk, i = e % dk;
        const float* pr = proj + (size_t)(row + j) * stride + (size_t)h * dk + i;
        Qs[j * ld + i] = j < cn ? pr[off_q] : 0.f;
        Ks[j * ld + i] = j < cn ? pr[off_k] : 0.f;
    }
    __syncthreads();
    {   // A: thread (ty, tx) computes rows 2 ty, 2 ty + 1 and columns 2 tx, 2 tx + 1
        const int ta = 2 * ty, ja = 2 * tx;
        float a00 = 0.f, a01 = 0.f, a10 = 0.f, a11 = 0.f;
        if (ja <= ta + 1) {
            const float* q0 = Qs + ta * ld;
            const float* k0 = Ks + ja * ld;
            for (int r = 0; r < dk; r++) {
                const float qa = q0[r], qb = q0[ld + r], ka = k0[r], kb = k0[ld + r];
                a00 = fmaf(qa, ka, a00); a01 = fmaf(qa, kb, a01);
                a10 = fmaf(qb, ka, a10); a11 = fmaf(qb, kb, a11);
            }
        }
        As[ta * (CC + 1) + ja] = ja <= ta ? a00 * pw[ta - ja] : 0.f;
        As[ta * (CC + 1) + ja + 1] = ja + 1 <= ta ? a01 * pw[ta - ja - 1] : 0.f;
        As[(ta + 1) * (CC + 1) + ja] = ja <= ta + 1 ? a10 * pw[ta + 1 - ja] : 0.f;
        As[(ta + 1) * (CC + 1) + ja + 1] = ja + 1 <= ta + 1 ? a11 * pw[ta - ja] : 0.f;
    }
    const float* Wg = W + ((size_t)blockIdx.x * H + h) * (size_t)dk * dv;
    const int t0 = 2 * ty, t1 = 2 * ty + 1;
    for (int cb = 0; cb < dv; cb += 128) {
        __syncthreads();                      // As is complete; the last pass has left Vs
        for (int e = tid; e < CC * 128; e += 256) {
            const int j = e / 128, i = e % 128;
            Vs[e] = (j < cn && cb + i < dv) ? proj[(size_t)(row + j) * stride + off_v + (size_t)h * dv + cb + i] : 0.f;
        }
        float acc0[8], acc1[8];
#pragma unroll
        for (int c = 0; c < 8; c++) { acc0[c] = 0.f; acc1[c] = 0.f; }
        for (int rb = 0; rb < dk; rb += 32) {
            __syncthreads();                  // the last block of S_before has been used (and Vs is there)
            for (int e = tid; e < 32 * 128; e += 256) {
                const int r = rb + e / 128, i = e % 128;
                Sb[e] = (r < dk && cb + i < dv) ? Wg[(size_t)r * dv + cb + i] : 0.f;
            }
            __syncthreads();
            const int rn = dk - rb < 32 ? dk - rb : 32;
            for (int r = 0; r < rn; r++) {
                const float qa = Qs[t0 * ld + rb + r], qb = Qs[t1 * ld + rb + r];
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    const float sv = Sb[r * 128 + tx + 16 * c];
                    acc0[c] = fmaf(qa, sv, acc0[c]);
                    acc1[c] = fmaf(qb, sv, acc1[c]);
                }
            }
        }
        const float g0 = pw[t0 + 1], g1 = pw[t1 + 1];
#pragma unroll
        for (int c = 0; c < 8; c++) { acc0[c] *= g0; acc1[c] *= g1; }
        for (int j = 0; j <= t1 && j < cn; j++) {
            const float a0 = As[t0 * (CC + 1) + j], a1 = As[t1 * (CC + 1) + j];
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float vv = Vs[j * 128 + tx + 16 * c];
                acc0[c] = fmaf(a0, vv, acc0[c]);
                acc1[c] = fmaf(a1, vv, acc1[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const int col = cb + tx + 16 * c;
            if (col >= dv) continue;
            if (t0 < cn) o[(size_t)(row + t0) * (size_t)(H * dv) + (size_t)h * dv + col] = acc0[c];
            if (t1 < cn) o[(size_t)(row + t1) * (size_t)(H * dv) + (size_t)h * dv + col] = acc1[c];
        }
    }
}

}  // namespace

extern "C" {

// The chunked form: four launches.  W is float32 scratch for max_chunks * H * dk * dv values; max_chunks is at least
// the number of chunks of CC = 32 tokens the step's sequences are cut into (tokens / 32 + sequences is enough).
// q and k are turned and scaled in place in proj.
int oe_retention_chunks(float* o, float* state, float* proj, long long stride, int off_q, int off_k, int off_v,
                        const float* cos_t, const float* sin_t, int rot, float k_scale, const float* decay,
                        const int* seq_slot, const int* cu_q, const int* tok_seq, const int* tok_pos, int n_tokens,
                        int n_seqs, int H, int dk, int dv, float* W, int max_chunks, cudaStream_t st) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (dk < 1 || dk > 256 || dv < 1 || H < 1 || H > 65535 || n_seqs > 65535 || rot < 0 || rot % 2 || rot > dk || max_chunks < 1)
        return OE_ERR_UNSUPPORTED;
    const size_t smem_state = sizeof(float) * (size_t)CC * (dk + dv);
    const size_t smem_out = sizeof(float) * ((size_t)2 * CC * (dk + 1) + CC * (CC + 1) + CC * 128 + 32 * 128 + CC + 1);
    if (smem_state > 200 * 1024) return OE_ERR_UNSUPPORTED;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(retention_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(retention_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    int rc = oe_launch(retention_prepare_kernel, dim3(n_tokens), dim3(128), 0, st, proj, stride, off_q, off_k, cos_t, sin_t, rot,
                       k_scale, tok_seq, tok_pos, H, dk);
    if (rc) return rc;
    rc = oe_launch(retention_chunk_state_kernel, dim3(max_chunks, H), dim3(256), smem_state, st, W, (const float*)proj, stride,
                   off_k, off_v, decay, cu_q, n_seqs, H, dk, dv);
    if (rc) return rc;
    rc = oe_launch(retention_chunk_carry_kernel, dim3((dk * dv + 255) / 256, H, n_seqs), dim3(256), 0, st, W, state, decay,
                   seq_slot, cu_q, H, dk, dv);
    if (rc) return rc;
    return oe_launch(retention_chunk_out_kernel, dim3(max_chunks, H), dim3(256), smem_out, st, o, (const float*)W,
                     (const float*)proj, stride, off_q, off_k, off_v, decay, cu_q, n_seqs, H, dk, dv);
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
