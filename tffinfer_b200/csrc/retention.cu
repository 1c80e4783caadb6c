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
// The token-by-token kernel (a CTA per (head, request), the state in shared memory) is the decode kernel: with one
// token a request it reads and writes the state once.  Portions of prompts run chunk by chunk: within a chunk of n
// tokens that starts from the state S_0
//   o_i = decay^(i+1) S_0^T q_i + sum_(j<=i) decay^(i-j) (q_i . k_j) v_j
//   S_n = decay^n S_0 + sum_j decay^(n-1-j) k_j v_j^T
// so the tokens of a chunk, and all chunks of a step, are worked on side by side, and only a cheap pass per state
// element walks the chunks in order.  Chunks are aligned to absolute positions of the request, so that the order of
// the additions that make a token's output depends on its position (and on where a portion was cut), not on what
// else is in the batch.
#include "common.cuh"
#include <type_traits>

namespace {

constexpr int NT = 256;

// four consecutive outputs in one store
template <typename T> __device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}

struct RetParams {
    const float* q; const float* k; float* vg; int ld, v_off, g_off;
    int clear;                         // v and g are set to zero behind the read (the rows are an accumulator buffer)
    float* state; int num_slots;
    const int* q_start; const int* pos_start; const int* slots;
    const float* decay;                // [H] on the device
    void* out; int H, d, dv; float eps;
};

// ------------------------------------------------------------------ token by token
// IN_SMEM: the head's state fits shared memory beside the rest (else it is worked on where it lies)
template <typename TO, bool IN_SMEM>
__global__ void __launch_bounds__(NT)
retention_step_kernel(RetParams p) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    const int d = p.d, dv = p.dv;
    float* S;
    if constexpr (IN_SMEM) S = sm;
    else S = p.state + ((size_t)min(max(p.slots[b], 0), p.num_slots - 1) * p.H + h) * d * dv;
    float* sq = sm + (IN_SMEM ? d * dv : 0);   // [d]
    float* sk = sq + d;                 // [d]
    float* sv = sk + d;                 // [dv]
    float* part = sv + dv;              // [NY][dv]
    const int JW = min(dv, NT);         // value columns worked on side by side, by NY groups of rows each
    const int NY = NT / JW;
    float* red = part + NY * dv;
    const int j0 = threadIdx.x % JW, ty = threadIdx.x / JW;
    const bool active = ty < NY;
    const int t0 = p.q_start[b], t1 = p.q_start[b + 1];
    const int slot = p.slots[b];
    const float decay = p.decay[h];
    pdl_wait();
    if (t1 <= t0 || slot < 0 || slot >= p.num_slots) return;
    float* gs = p.state + ((size_t)slot * p.H + h) * d * dv;
    if (IN_SMEM) for (int e = threadIdx.x; e < d * dv; e += NT) S[e] = gs[e];
    for (int t = t0; t < t1; ++t) {
        __syncthreads();
        for (int i = threadIdx.x; i < d; i += NT) {
            sq[i] = p.q[(size_t)t * p.H * d + (size_t)h * d + i];
            sk[i] = p.k[(size_t)t * p.H * d + (size_t)h * d + i];
        }
        for (int i = threadIdx.x; i < dv; i += NT) {
            sv[i] = p.vg[(size_t)t * p.ld + p.v_off + h * dv + i];
            if (p.clear) p.vg[(size_t)t * p.ld + p.v_off + h * dv + i] = 0.f;
        }
        __syncthreads();
        if (active) {
            for (int j = j0; j < dv; j += JW) {
                float acc = 0.f;
                const float vj = sv[j];
                for (int i = ty; i < d; i += NY) {
                    const float s = fmaf(decay, S[i * dv + j], sk[i] * vj);
                    S[i * dv + j] = s;
                    acc = fmaf(s, sq[i], acc);
                }
                part[ty * dv + j] = acc;
            }
        }
        __syncthreads();
        float sq_sum = 0.f;
        for (int j = threadIdx.x; j < dv; j += NT) {
            float o = 0.f;
            for (int y = 0; y < NY; ++y) o += part[y * dv + j];
            part[j] = o;                                          // row 0 now holds the outputs (only this thread reads column j)
            sq_sum = fmaf(o, o, sq_sum);
        }
        const float ss = block_sum<NT>(sq_sum, red);
        const float rs = rsqrtf(ss / (float)dv + p.eps);
        for (int j = threadIdx.x; j < dv; j += NT) {
            const float g = p.vg[(size_t)t * p.ld + p.g_off + h * dv + j];
            if (p.clear) p.vg[(size_t)t * p.ld + p.g_off + h * dv + j] = 0.f;
            ((TO*)p.out)[(size_t)t * p.H * dv + (size_t)h * dv + j] = from_f32<TO>((part[j] * rs) * (g / (1.0f + expf(-g))));
        }
    }
    __syncthreads();
    if (IN_SMEM) for (int e = threadIdx.x; e < d * dv; e += NT) gs[e] = S[e];
}

// ------------------------------------------------------------------ chunk by chunk
// Portions of prompts.  A chunk is up to C tokens of one request that do not cross a multiple of C of the request's
// positions.  Three kernels, the first and the last with a CTA per (chunk, head), so that all chunks of a prompt are
// worked on at once:
//   1. local:  A = mask(decay^(i-j) q_i . k_j);  acc = A V  (-> acc [T, H*dv]);  U = sum_j decay^(n-1-j) k_j v_j^T (-> U[chunk])
//   2. scan:   per (request, head, state element), over the request's chunks in order: U[chunk] <- S (the state the
//              chunk starts from), S <- decay^n S + U[chunk]; the last S goes back to the request's slot
//   3. finish: o_i = acc_i + decay^(i+1) S^T q_i (S in blocks of 64 value columns), then the head's RMS norm and
//              the gate -> out
// The products are float32 FMAs on 4 x 4 register tiles out of shared memory (operands zero-padded to multiples of 4).
constexpr int C = 64;

__host__ __device__ inline int pad4(int x) { return (x + 3) & ~3; }

// Which chunk is CTA ``index``: request b, first row t, tokens n, position of the first token; false beyond the last.
struct ChunkRef { int b, t, n, pos; };
__device__ inline bool find_chunk(const RetParams& p, int num_requests, int index, ChunkRef& c) {
    for (int b = 0; b < num_requests; ++b) {
        const int t0 = p.q_start[b], len = p.q_start[b + 1] - t0;
        if (len <= 0) continue;
        const int pos0 = p.pos_start[b];
        const int first = pos0 / C, count = (pos0 + len - 1) / C - first + 1;
        if (index < count) {
            const int lo = max(pos0, (first + index) * C), hi = min(pos0 + len, (first + index + 1) * C);
            c.b = b; c.pos = lo; c.t = t0 + (lo - pos0); c.n = hi - lo;
            return true;
        }
        index -= count;
    }
    return false;
}

// out(m, n) = sum_k A[m][k] B[k][n] for m < M, n < N; K a multiple of 4; rows of A up to pad4(M) and columns of B up
// to pad4(N) are readable.  Consecutive threads take consecutive column tiles.
// ``lower``: 0 = nothing known; 1 = only outputs with n <= m are wanted (tiles above the diagonal are left out);
// 2 = A is lower triangular (A[m][k] = 0 for k > m: the sum stops at the tile's last row).
template <typename F>
__device__ __forceinline__ void tile_product(const float* __restrict__ A, int lda, const float* __restrict__ B, int ldb,
                                             int M, int N, int K, F&& store, int lower = 0) {
    const int tn = (N + 3) >> 2, tm = (M + 3) >> 2;
    for (int tile = threadIdx.x; tile < tm * tn; tile += NT) {
        const int m0 = (tile / tn) << 2, n0 = (tile % tn) << 2;
        if (lower == 1 && n0 > m0 + 3) continue;
        const int kend = lower == 2 ? min(K, m0 + 4) : K;
        float acc[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
        for (int k = 0; k < kend; k += 4) {
            float4 a[4], b[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) a[r] = *reinterpret_cast<const float4*>(A + (m0 + r) * lda + k);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) b[kk] = *reinterpret_cast<const float4*>(B + (k + kk) * ldb + n0);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float av[4] = {a[r].x, a[r].y, a[r].z, a[r].w};
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    acc[r][0] = fmaf(av[kk], b[kk].x, acc[r][0]);
                    acc[r][1] = fmaf(av[kk], b[kk].y, acc[r][1]);
                    acc[r][2] = fmaf(av[kk], b[kk].z, acc[r][2]);
                    acc[r][3] = fmaf(av[kk], b[kk].w, acc[r][3]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (m0 + r < M && n0 + c < N) store(m0 + r, n0 + c, acc[r][c]);
    }
}

__device__ __forceinline__ void fill_powers(float* pw, float decay) {
    if (threadIdx.x == 0) { float x = 1.f; for (int i = 0; i <= C; ++i) { pw[i] = x; x *= decay; } }
}

__global__ void __launch_bounds__(NT)
retention_local_kernel(RetParams p, int num_requests, float* __restrict__ acc, float* __restrict__ U) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float pw[C + 1];
    pdl_launch_dependents();
    const int h = blockIdx.y, d = p.d, dv = p.dv, dP = pad4(d), vP = pad4(dv);
    float* sq = sm;                      // [C][dP]
    float* skT = sq + C * dP;            // [dP][C]
    float* sv = skT + dP * C;            // [C][vP]
    float* sA = sv + C * vP;             // [C][C]
    ChunkRef c;
    const bool have = find_chunk(p, num_requests, blockIdx.x, c);
    fill_powers(pw, p.decay[h]);
    pdl_wait();
    if (!have) return;
    const int n = c.n, nP = pad4(n);
    for (int e = threadIdx.x; e < C * dP + dP * C + C * vP + C * C; e += NT) sm[e] = 0.f;
    __syncthreads();
    for (int e = threadIdx.x; e < n * d; e += NT) {
        const int i = e / d, r = e % d;
        sq[i * dP + r] = p.q[(size_t)(c.t + i) * p.H * d + (size_t)h * d + r];
        skT[r * C + i] = p.k[(size_t)(c.t + i) * p.H * d + (size_t)h * d + r];
    }
    for (int e = threadIdx.x; e < n * dv; e += NT) {
        const int i = e / dv, r = e % dv;
        sv[i * vP + r] = p.vg[(size_t)(c.t + i) * p.ld + p.v_off + h * dv + r];
        if (p.clear) p.vg[(size_t)(c.t + i) * p.ld + p.v_off + h * dv + r] = 0.f;
    }
    __syncthreads();
    // (sA was cleared above: the tiles above the diagonal, which are left out, hold zeros)
    tile_product(sq, dP, skT, C, n, n, dP, [&](int i, int j, float a) { sA[i * C + j] = j <= i ? a * pw[i - j] : 0.f; }, 1);
    __syncthreads();
    tile_product(sA, C, sv, vP, n, dv, nP, [&](int i, int r, float a) {
        acc[(size_t)(c.t + i) * p.H * dv + (size_t)h * dv + r] = a;
    }, 2);
    __syncthreads();                                                  // every thread is done with skT as it was
    for (int e = threadIdx.x; e < d * n; e += NT) { const int r = e / n, j = e % n; skT[r * C + j] *= pw[n - 1 - j]; }
    __syncthreads();
    float* Uc = U + ((size_t)blockIdx.x * p.H + h) * d * dv;
    tile_product(skT, C, sv, vP, d, dv, nP, [&](int r, int cc, float a) { Uc[r * dv + cc] = a; });
}

// VEC = 4: a thread walks four neighbouring state elements (16-byte accesses); 1: one element.
template <int VEC>
__global__ void __launch_bounds__(NT)
retention_scan_kernel(RetParams p, int num_requests, float* __restrict__ U) {
    pdl_launch_dependents();
    const int h = blockIdx.y, b = blockIdx.z;
    const int e = (blockIdx.x * NT + threadIdx.x) * VEC;
    const int t0 = p.q_start[b], len = p.q_start[b + 1] - t0;
    const int slot = p.slots[b];
    const float decay = p.decay[h];
    int first_chunk = 0;                                               // chunks of the requests ahead of b
    for (int r = 0; r < b; ++r) {
        const int l = p.q_start[r + 1] - p.q_start[r];
        if (l > 0) first_chunk += (p.pos_start[r] + l - 1) / C - p.pos_start[r] / C + 1;
    }
    pdl_wait();
    if (len <= 0 || slot < 0 || slot >= p.num_slots || e >= p.d * p.dv) return;
    const int pos0 = p.pos_start[b];
    const int count = (pos0 + len - 1) / C - pos0 / C + 1;
    typedef typename std::conditional<VEC == 4, float4, float>::type V;
    V* gs = reinterpret_cast<V*>(p.state + ((size_t)slot * p.H + h) * p.d * p.dv + e);
    V S = *gs;
    const size_t stride = (size_t)p.H * p.d * p.dv / VEC;             // V's between a chunk's U and the next one's
    V* u0 = reinterpret_cast<V*>(U + ((size_t)first_chunk * p.H + h) * p.d * p.dv + e);
    float g_full = 1.f;
    for (int i = 0; i < C; ++i) g_full *= decay;                       // the same product as the other kernels' table
    // eight chunks' U are asked for together, then the state walks through them: the loads of a chunk do not wait
    // for the chunk before
    for (int c0 = 0; c0 < count; c0 += 8) {
        V add[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) if (c0 + j < count) add[j] = u0[(size_t)(c0 + j) * stride];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = c0 + j;
            if (c < count) {
                const int lo = max(pos0, (pos0 / C + c) * C), hi = min(pos0 + len, (pos0 / C + c + 1) * C);
                u0[(size_t)c * stride] = S;
                float g = g_full;
                if (hi - lo != C) { g = 1.f; for (int i = 0; i < hi - lo; ++i) g *= decay; }
                if constexpr (VEC == 4) {
                    S.x = fmaf(g, S.x, add[j].x); S.y = fmaf(g, S.y, add[j].y);
                    S.z = fmaf(g, S.z, add[j].z); S.w = fmaf(g, S.w, add[j].w);
                } else {
                    S = fmaf(g, S, add[j]);
                }
            }
        }
    }
    *gs = S;
}

// The value columns are worked on in blocks of NB, so that the CTA holds q, one block of S and the outputs (96 KB
// at 128 x 128: two CTAs an SM, one loading while the other multiplies).
constexpr int NB = 64;

template <typename TO>
__global__ void __launch_bounds__(NT)
retention_finish_kernel(RetParams p, int num_requests, const float* __restrict__ acc, const float* __restrict__ U) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float pw[C + 1];
    __shared__ float srs[C];             // the rows' 1 / rms
    pdl_launch_dependents();
    const int h = blockIdx.y, d = p.d, dv = p.dv, dP = pad4(d), vP = pad4(dv);
    float* sq = sm;                      // [C][dP]
    float* sS = sq + C * dP;             // [dP][NB]
    float* so = sS + dP * NB;            // [C][vP]
    ChunkRef c;
    const bool have = find_chunk(p, num_requests, blockIdx.x, c);
    fill_powers(pw, p.decay[h]);
    pdl_wait();
    if (!have) return;
    const int n = c.n;
    const float* Sc = U + ((size_t)blockIdx.x * p.H + h) * d * dv;
    const float* qg = p.q + (size_t)c.t * p.H * d + (size_t)h * d;
    // rows of four: 16-byte loads when every row starts on such a boundary
    const bool vec = (d & 3) == 0 && (dv & 3) == 0 && (((uintptr_t)p.q | (uintptr_t)U) & 15) == 0;
    if (vec) {
        const int d4 = d >> 2;
        for (int e = threadIdx.x; e < pad4(n) * d4; e += NT) {
            const int i = e / d4, r = e % d4;
            reinterpret_cast<float4*>(sq + i * dP)[r] =
                i < n ? reinterpret_cast<const float4*>(qg + (size_t)i * p.H * d)[r] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    } else {
        for (int e = threadIdx.x; e < C * dP; e += NT) sq[e] = 0.f;
        __syncthreads();
        for (int e = threadIdx.x; e < n * d; e += NT) sq[(e / d) * dP + e % d] = qg[(size_t)(e / d) * p.H * d + e % d];
    }
    // the chunk's local part goes into the output tile first (the product below adds to it): loads asked for together
    // here, not one by one between the product's stores
    const float* ag = acc + (size_t)c.t * p.H * dv + (size_t)h * dv;
    if (vec && (((uintptr_t)acc) & 15) == 0) {
        const int v4 = dv >> 2;
        for (int e = threadIdx.x; e < n * v4; e += NT)
            reinterpret_cast<float4*>(so + (e / v4) * vP)[e % v4] = reinterpret_cast<const float4*>(ag + (size_t)(e / v4) * p.H * dv)[e % v4];
    } else {
        for (int e = threadIdx.x; e < n * dv; e += NT) so[(e / dv) * vP + e % dv] = ag[(size_t)(e / dv) * p.H * dv + e % dv];
    }
    for (int n0 = 0; n0 < dv; n0 += NB) {
        const int nb = min(NB, dv - n0);
        __syncthreads();                                              // the block before has been multiplied
        if (vec) {
            const int b4 = nb >> 2;
            for (int e = threadIdx.x; e < d * b4; e += NT) {
                const int r = e / b4, cc = e % b4;
                reinterpret_cast<float4*>(sS + r * NB)[cc] = reinterpret_cast<const float4*>(Sc + (size_t)r * dv + n0)[cc];
            }
        } else {
            for (int e = threadIdx.x; e < dP * NB; e += NT) {
                const int r = e / NB, cc = e % NB;
                sS[e] = (r < d && cc < nb) ? Sc[(size_t)r * dv + n0 + cc] : 0.f;
            }
        }
        __syncthreads();
        tile_product(sq, dP, sS, NB, n, nb, dP, [&](int i, int r, float a) {
            so[i * vP + n0 + r] = fmaf(pw[i + 1], a, so[i * vP + n0 + r]);
        });
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* gg = p.vg + (size_t)c.t * p.ld + p.g_off + h * dv;         // the chunk's gates, rows ld apart
    if (vec && (p.ld & 3) == 0 && (((uintptr_t)gg | (uintptr_t)p.out) & 15) == 0) {
        // the rows' scales, a warp per token, then all elements with the gates asked for eight loads at a time
        for (int i = warp; i < n; i += NT / 32) {
            float ss = 0.f;
            for (int r = lane; r < dv; r += 32) ss = fmaf(so[i * vP + r], so[i * vP + r], ss);
            ss = warp_sum(ss);
            if (lane == 0) srs[i] = rsqrtf(ss / (float)dv + p.eps);
        }
        __syncthreads();
        const int v4 = dv >> 2, total4 = n * v4;
        TO* og = (TO*)p.out + (size_t)c.t * p.H * dv + (size_t)h * dv;
        for (int e0 = threadIdx.x; e0 < total4; e0 += NT * 8) {
            float4 g[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int e = e0 + k * NT;
                if (e < total4) g[k] = reinterpret_cast<const float4*>(gg + (size_t)(e / v4) * p.ld)[e % v4];
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int e = e0 + k * NT;
                if (e < total4) {
                    const int i = e / v4, r4 = e % v4;
                    if (p.clear) reinterpret_cast<float4*>(gg + (size_t)i * p.ld)[r4] = make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 o = reinterpret_cast<const float4*>(so + i * vP)[r4];
                    const float rs = srs[i];
                    store4<TO>(og + (size_t)i * p.H * dv + 4 * r4,
                               (o.x * rs) * (g[k].x / (1.0f + expf(-g[k].x))), (o.y * rs) * (g[k].y / (1.0f + expf(-g[k].y))),
                               (o.z * rs) * (g[k].z / (1.0f + expf(-g[k].z))), (o.w * rs) * (g[k].w / (1.0f + expf(-g[k].w))));
                }
            }
        }
        return;
    }
    for (int i = warp; i < n; i += NT / 32) {                         // the rows' norms and gates: a warp per token
        float ss = 0.f;
        for (int r = lane; r < dv; r += 32) ss = fmaf(so[i * vP + r], so[i * vP + r], ss);
        ss = warp_sum(ss);
        const float rs = rsqrtf(ss / (float)dv + p.eps);
        for (int r = lane; r < dv; r += 32) {
            const float g = p.vg[(size_t)(c.t + i) * p.ld + p.g_off + h * dv + r];
            if (p.clear) p.vg[(size_t)(c.t + i) * p.ld + p.g_off + h * dv + r] = 0.f;
            ((TO*)p.out)[(size_t)(c.t + i) * p.H * dv + (size_t)h * dv + r] =
                from_f32<TO>((so[i * vP + r] * rs) * (g / (1.0f + expf(-g))));
        }
    }
}

}  // namespace

// Floats of workspace the chunked form needs for a step of ``num_tokens`` tokens in ``num_requests`` requests.
TFF_API long long tff_retention_workspace(int num_tokens, int num_requests, int H, int d, int dv) {
    const long long chunks = num_tokens / C + 2ll * num_requests;
    return (long long)num_tokens * H * dv + chunks * H * d * dv;
}

// clear_vg != 0: the v and g columns of ``vg`` are set to zero once read.
// chunked != 0: chunk by chunk (portions of prompts; ``workspace`` of tff_retention_workspace floats, ``num_tokens``
// the step's tokens); else token by token (decoded tokens).  TFF_ERR_UNSUPPORTED when a head does not fit the
// shared memory of the form asked for.
TFF_API int tff_retention(
    const float* q, const float* k, float* vg, int clear_vg, int ld, int v_off, int g_off,
    float* state, int num_slots, const int* q_start, const int* pos_start, const int* slots, const float* decay,
    void* out, int out_is_bf16, int num_requests, int H, int d, int dv, float eps, int chunked,
    float* workspace, int num_tokens, cudaStream_t stream) {
    if (num_requests <= 0) return TFF_OK;
    if (!q || !k || !vg || !state || !q_start || !pos_start || !slots || !decay || !out || H <= 0 || d <= 0 || dv <= 0)
        return TFF_ERR_BAD_ARGUMENT;
    if (num_requests > 65535 || H > 65535) return TFF_ERR_UNSUPPORTED;
    RetParams p;
    p.q = q; p.k = k; p.vg = vg; p.clear = clear_vg; p.ld = ld; p.v_off = v_off; p.g_off = g_off;
    p.state = state; p.num_slots = num_slots; p.q_start = q_start; p.pos_start = pos_start; p.slots = slots;
    p.decay = decay; p.out = out; p.H = H; p.d = d; p.dv = dv; p.eps = eps;
    constexpr size_t MOST = 224 * 1024;        // dynamic shared memory a CTA may ask for here (the kernels have a little static on top)
    if (chunked) {
        if (!workspace || num_tokens <= 0) return TFF_ERR_BAD_ARGUMENT;
        const int dP = pad4(d), vP = pad4(dv);
        const size_t smem1 = sizeof(float) * ((size_t)C * dP + (size_t)dP * C + (size_t)C * vP + (size_t)C * C);
        const size_t smem3 = sizeof(float) * ((size_t)C * dP + (size_t)dP * NB + (size_t)C * vP);
        if (smem1 > MOST || smem3 > MOST) return TFF_ERR_UNSUPPORTED;
        const int chunks = num_tokens / C + 2 * num_requests;
        float* acc = workspace;
        float* U = workspace + (size_t)num_tokens * H * dv;
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(retention_local_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MOST) != cudaSuccess ||
                cudaFuncSetAttribute(retention_finish_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MOST) != cudaSuccess ||
                cudaFuncSetAttribute(retention_finish_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MOST) != cudaSuccess)
                return TFF_ERR_LAUNCH;
            configured = true;
        }
        int st = tff_launch_pdl(retention_local_kernel, dim3(chunks, H), dim3(NT), smem1, stream, p, num_requests, acc, U);
        if (st != TFF_OK) return st;
        if ((d * dv) % 4 == 0 && ((uintptr_t)state & 15) == 0 && ((uintptr_t)U & 15) == 0)
            st = tff_launch_pdl(retention_scan_kernel<4>, dim3((d * dv / 4 + NT - 1) / NT, H, num_requests), dim3(NT), (size_t)0,
                                stream, p, num_requests, U);
        else
            st = tff_launch_pdl(retention_scan_kernel<1>, dim3((d * dv + NT - 1) / NT, H, num_requests), dim3(NT), (size_t)0,
                                stream, p, num_requests, U);
        if (st != TFF_OK) return st;
        if (out_is_bf16)
            return tff_launch_pdl(retention_finish_kernel<bf16>, dim3(chunks, H), dim3(NT), smem3, stream, p, num_requests,
                                  (const float*)acc, (const float*)U);
        return tff_launch_pdl(retention_finish_kernel<float>, dim3(chunks, H), dim3(NT), smem3, stream, p, num_requests,
                              (const float*)acc, (const float*)U);
    }
    const size_t rest = sizeof(float) * ((size_t)2 * d + dv + (size_t)(NT / (dv < NT ? dv : NT)) * dv + 32);
    const int in_smem = sizeof(float) * (size_t)d * dv + rest <= MOST ? 1 : 0;
    const size_t smem = rest + (in_smem ? sizeof(float) * (size_t)d * dv : 0);
    if (smem > MOST) return TFF_ERR_UNSUPPORTED;
    {
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(retention_step_kernel<bf16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MOST) != cudaSuccess ||
                cudaFuncSetAttribute(retention_step_kernel<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MOST) != cudaSuccess)
                return TFF_ERR_LAUNCH;
            configured = true;
        }
    }
    const dim3 grid(H, num_requests);
    if (in_smem) {
        if (out_is_bf16) return tff_launch_pdl(retention_step_kernel<bf16, true>, grid, dim3(NT), smem, stream, p);
        return tff_launch_pdl(retention_step_kernel<float, true>, grid, dim3(NT), smem, stream, p);
    }
    if (out_is_bf16) return tff_launch_pdl(retention_step_kernel<bf16, false>, grid, dim3(NT), smem, stream, p);
    return tff_launch_pdl(retention_step_kernel<float, false>, grid, dim3(NT), smem, stream, p);
}
