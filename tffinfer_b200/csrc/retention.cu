// Retention: linear attention with a fixed decay per head, no softmax and no denominator, over a per-request
// state kept in float32.
//   S_t = decay_h S_(t-1) + k_t v_t^T          S [d, dv] per (request, head), zero before the first token
//   o_t = S_t^T q_t
//   out_t = o_t * rsqrt(mean_j(o_t[j]^2) + eps) * silu(g_t)      (per head; silu(g) = g / (1 + exp(-g)))
// q, k [T, H*d] float32, already rotated (k already scaled); v and g are read from a float32 row of stride ld
// (the mixer's merged projection) at offsets v_off and g_off; out [T, H*dv] in the activation type.
// state [slots, H, d, dv] float32; request b of the step uses slot slots[b] and brings the rows
// q_start[b] .. q_start[b+1]-1.  Everything is float32 FMA.
//
// Two kernels.  The token-by-token one (a CTA per (head, request), the state in shared memory) is the decode
// kernel: with one token a request it reads and writes the state once.  Portions of prompts run chunk by chunk:
// within a chunk of C tokens
//   o_i = decay^(i+1) S_0^T q_i + sum_(j<=i) decay^(i-j) (q_i . k_j) v_j
//   S_C = decay^C S_0 + sum_j decay^(C-1-j) k_j v_j^T
// so the C tokens of a chunk are worked on side by side and the state is touched once a chunk.  Chunks are aligned
// to absolute positions of the request (a chunk never crosses a multiple of C), so that the order of the
// additions that make a token's output depends on its position alone, not on how the prompt was cut.
#include "common.cuh"

namespace {

constexpr int NT = 256;

struct RetParams {
    const float* q; const float* k; const float* vg; int ld, v_off, g_off;
    float* state; int num_slots;
    const int* q_start; const int* pos_start; const int* slots;
    const float* decay;                // [H] on the device
    void* out; int H, d, dv; float eps;
};

// ------------------------------------------------------------------ token by token
template <typename TO>
__global__ void __launch_bounds__(NT)
retention_step_kernel(RetParams p) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    const int d = p.d, dv = p.dv;
    float* S = sm;                      // [d][dv]
    float* sq = S + d * dv;             // [d]
    float* sk = sq + d;                 // [d]
    float* sv = sk + d;                 // [dv]
    float* part = sv + dv;              // [NY][dv]
    float* red = part + (NT / 1) ;      // generous: NY * dv <= NT
    const int NY = NT / dv > 0 ? NT / dv : 1;
    const int j = threadIdx.x % dv, ty = threadIdx.x / dv;
    const bool active = ty < NY && dv <= NT;
    const int t0 = p.q_start[b], t1 = p.q_start[b + 1];
    const int slot = p.slots[b];
    const float decay = p.decay[h];
    pdl_wait();
    if (t1 <= t0 || slot < 0 || slot >= p.num_slots) return;
    float* gs = p.state + ((size_t)slot * p.H + h) * d * dv;
    for (int e = threadIdx.x; e < d * dv; e += NT) S[e] = gs[e];
    for (int t = t0; t < t1; ++t) {
        __syncthreads();
        for (int i = threadIdx.x; i < d; i += NT) {
            sq[i] = p.q[(size_t)t * p.H * d + (size_t)h * d + i];
            sk[i] = p.k[(size_t)t * p.H * d + (size_t)h * d + i];
        }
        for (int i = threadIdx.x; i < dv; i += NT) sv[i] = p.vg[(size_t)t * p.ld + p.v_off + h * dv + i];
        __syncthreads();
        if (active) {
            float acc = 0.f;
            const float vj = sv[j];
            for (int i = ty; i < d; i += NY) {
                const float s = fmaf(decay, S[i * dv + j], sk[i] * vj);
                S[i * dv + j] = s;
                acc = fmaf(s, sq[i], acc);
            }
            part[ty * dv + j] = acc;
        }
        __syncthreads();
        float o = 0.f;
        if (threadIdx.x < dv) for (int y = 0; y < NY; ++y) o += part[y * dv + threadIdx.x];
        const float ss = block_sum<NT>(threadIdx.x < dv ? o * o : 0.f, red);
        if (threadIdx.x < dv) {
            const float rs = rsqrtf(ss / (float)dv + p.eps);
            const float g = p.vg[(size_t)t * p.ld + p.g_off + h * dv + threadIdx.x];
            ((TO*)p.out)[(size_t)t * p.H * dv + (size_t)h * dv + threadIdx.x] =
                from_f32<TO>((o * rs) * (g / (1.0f + expf(-g))));
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < d * dv; e += NT) gs[e] = S[e];
}

// ------------------------------------------------------------------ chunk by chunk
// A CTA per (head, request).  Shared memory: the state [d][dv], and of the chunk q [C][d+1], k [C][d+1],
// v [C][dv], the masked, decayed scores A [C][C+1] and the powers of the decay.
constexpr int C = 32;

template <typename TO>
__global__ void __launch_bounds__(NT)
retention_chunk_kernel(RetParams p) {
    extern __shared__ float sm[];
    __shared__ float pw[C + 1];         // decay^0 .. decay^C
    __shared__ float red[32];
    pdl_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    const int d = p.d, dv = p.dv, dq = d + 1;
    float* S = sm;                      // [d][dv]
    float* sq = S + d * dv;             // [C][d+1]
    float* sk = sq + C * dq;            // [C][d+1]
    float* sv = sk + C * dq;            // [C][dv]
    float* A = sv + C * dv;             // [C][C+1]
    float* so = A + C * (C + 1);        // [C][dv]
    const int t0 = p.q_start[b], t1 = p.q_start[b + 1];
    const int pos0 = p.pos_start[b];
    const int slot = p.slots[b];
    const float decay = p.decay[h];
    if (threadIdx.x == 0) { float x = 1.f; for (int i = 0; i <= C; ++i) { pw[i] = x; x *= decay; } }
    pdl_wait();
    if (t1 <= t0 || slot < 0 || slot >= p.num_slots) return;
    float* gs = p.state + ((size_t)slot * p.H + h) * d * dv;
    for (int e = threadIdx.x; e < d * dv; e += NT) S[e] = gs[e];
    int t = t0;
    while (t < t1) {
        const int pos = pos0 + (t - t0);
        const int n = min(t1 - t, C - pos % C);                 // tokens of this chunk (ends at a multiple of C)
        __syncthreads();
        for (int e = threadIdx.x; e < n * d; e += NT) {
            const int i = e / d, c = e % d;
            sq[i * dq + c] = p.q[(size_t)(t + i) * p.H * d + (size_t)h * d + c];
            sk[i * dq + c] = p.k[(size_t)(t + i) * p.H * d + (size_t)h * d + c];
        }
        for (int e = threadIdx.x; e < n * dv; e += NT) {
            const int i = e / dv, c = e % dv;
            sv[e] = p.vg[(size_t)(t + i) * p.ld + p.v_off + h * dv + c];
        }
        __syncthreads();
        // A[i][j] = decay^(i-j) (q_i . k_j) for j <= i
        for (int e = threadIdx.x; e < n * n; e += NT) {
            const int i = e / n, jj = e % n;
            float a = 0.f;
            if (jj <= i) {
                for (int c = 0; c < d; ++c) a = fmaf(sq[i * dq + c], sk[jj * dq + c], a);
                a *= pw[i - jj];
            }
            A[i * (C + 1) + jj] = a;
        }
        __syncthreads();
        // o[i][c] = decay^(i+1) sum_r q_i[r] S[r][c] + sum_(j<=i) A[i][j] v_j[c]
        for (int e = threadIdx.x; e < n * dv; e += NT) {
            const int i = e / dv, c = e % dv;
            float a = 0.f;
            for (int r = 0; r < d; ++r) a = fmaf(sq[i * dq + r], S[r * dv + c], a);
            a *= pw[i + 1];
            for (int jj = 0; jj <= i; ++jj) a = fmaf(A[i * (C + 1) + jj], sv[jj * dv + c], a);
            so[e] = a;
        }
        __syncthreads();
        // S = decay^n S + sum_j decay^(n-1-j) k_j v_j^T
        for (int e = threadIdx.x; e < d * dv; e += NT) {
            const int r = e / dv, c = e % dv;
            float a = S[e] * pw[n];
            for (int jj = 0; jj < n; ++jj) a = fmaf(sk[jj * dq + r] * pw[n - 1 - jj], sv[jj * dv + c], a);
            S[e] = a;
        }
        // the rows' norms and gates: a warp per token
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int i = warp; i < n; i += NT / 32) {
            float ss = 0.f;
            for (int c = lane; c < dv; c += 32) ss = fmaf(so[i * dv + c], so[i * dv + c], ss);
            ss = warp_sum(ss);
            const float rs = rsqrtf(ss / (float)dv + p.eps);
            for (int c = lane; c < dv; c += 32) {
                const float g = p.vg[(size_t)(t + i) * p.ld + p.g_off + h * dv + c];
                ((TO*)p.out)[(size_t)(t + i) * p.H * dv + (size_t)h * dv + c] =
                    from_f32<TO>((so[i * dv + c] * rs) * (g / (1.0f + expf(-g))));
            }
        }
        t += n;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < d * dv; e += NT) gs[e] = S[e];
    (void)red;
}

}  // namespace

// chunked != 0: the chunk-by-chunk kernel (portions of prompts); else token by token (decoded tokens).
TFF_API int tff_retention(
    const float* q, const float* k, const float* vg, int ld, int v_off, int g_off,
    float* state, int num_slots, const int* q_start, const int* pos_start, const int* slots, const float* decay,
    void* out, int out_is_bf16, int num_requests, int H, int d, int dv, float eps, int chunked, cudaStream_t stream) {
    if (num_requests <= 0) return TFF_OK;
    if (!q || !k || !vg || !state || !q_start || !pos_start || !slots || !decay || !out || H <= 0 || d <= 0 || dv <= 0)
        return TFF_ERR_BAD_ARGUMENT;
    if (dv > NT || num_requests > 65535) return TFF_ERR_UNSUPPORTED;
    RetParams p;
    p.q = q; p.k = k; p.vg = vg; p.ld = ld; p.v_off = v_off; p.g_off = g_off;
    p.state = state; p.num_slots = num_slots; p.q_start = q_start; p.pos_start = pos_start; p.slots = slots;
    p.decay = decay; p.out = out; p.H = H; p.d = d; p.dv = dv; p.eps = eps;
    size_t smem;
    if (chunked) smem = sizeof(float) * ((size_t)d * dv + 2 * (size_t)C * (d + 1) + 2 * (size_t)C * dv + C * (C + 1));
    else smem = sizeof(float) * ((size_t)d * dv + 2 * d + dv + NT + 32);
    if (smem > 200 * 1024) return TFF_ERR_UNSUPPORTED;
#define TFF_RET(KERN)                                                                                              \
    do {                                                                                                           \
        auto kern = KERN;                                                                                          \
        static bool configured = false;                                                                            \
        if (!configured) {                                                                                         \
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) \
                return TFF_ERR_LAUNCH;                                                                             \
            configured = true;                                                                                     \
        }                                                                                                          \
        return tff_launch_pdl(kern, dim3(H, num_requests), dim3(NT), smem, stream, p);                             \
    } while (0)
    if (chunked) {
        if (out_is_bf16) TFF_RET(retention_chunk_kernel<bf16>);
        TFF_RET(retention_chunk_kernel<float>);
    }
    if (out_is_bf16) TFF_RET(retention_step_kernel<bf16>);
    TFF_RET(retention_step_kernel<float>);
#undef TFF_RET
}
