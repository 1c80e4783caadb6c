// minGRU: a gated recurrence whose gates read only the current token, over a float32 state of ``width`` elements per
// request.  From the float32 accumulators of the input projection, row t = [.. z (width) .. x (width) .. g (width) ..]:
//   z_t = sigmoid(z + bz)        u_t = x + bx        c_t = u_t + 1/2 where u_t >= 0, sigmoid(u_t) where u_t < 0
//   S_t = (1 - z_t) S_(t-1) + z_t c_t           element by element, S before a request's first token = its state slot
//   out_t = out_scale * S_t * silu(g)
// One thread per (request, channel) walks the request's tokens of this step in order and leaves the last S in the
// slot; everything is float32 and only the store of out rounds.  With ``clear_input`` the three inputs are set to zero
// behind the read (the row is then an accumulator buffer that the next split product adds into).
#include "common.cuh"

namespace {

template <typename TO>
__global__ void __launch_bounds__(128)
min_gru_kernel(float* __restrict__ proj, int ld, int z_off, int x_off, int g_off, int clear_input,
               const float* __restrict__ bz, const float* __restrict__ bx, float* __restrict__ state,
               const int* __restrict__ q_start, const int* __restrict__ slots, int width,
               TO* __restrict__ out, int out_ld, int out_off, float out_scale) {
    pdl_launch_dependents();
    const int c = blockIdx.x * 128 + threadIdx.x, b = blockIdx.y;
    if (c >= width) return;
    const float bzc = bz ? bz[c] : 0.f, bxc = bx ? bx[c] : 0.f;
    pdl_wait();
    const int t0 = q_start[b], t1 = q_start[b + 1];
    float* sp = state + (size_t)slots[b] * width + c;
    float S = *sp;
    for (int t = t0; t < t1; ++t) {
        float* row = proj + (size_t)t * ld;
        const float zr = row[z_off + c], xr = row[x_off + c], gr = row[g_off + c];
        if (clear_input) { row[z_off + c] = 0.f; row[x_off + c] = 0.f; row[g_off + c] = 0.f; }
        const float z = 1.0f / (1.0f + expf(-(zr + bzc)));
        const float u = xr + bxc;
        const float cand = u >= 0.f ? u + 0.5f : 1.0f / (1.0f + expf(-u));
        S = (1.0f - z) * S + z * cand;
        const float gate = gr / (1.0f + expf(-gr));
        out[(size_t)t * out_ld + out_off + c] = from_f32<TO>(out_scale * S * gate);
    }
    *sp = S;
}

// The same recurrence for long portions, in chunks of CHUNK tokens of a request that are worked on side by side.  With
// a_t = 1 - z_t and b_t = z_t c_t the recurrence is S_t = a_t S_(t-1) + b_t, so a chunk maps its incoming state to
// A S + B with A = prod a_t and B = the chunk run from zero:
//   pass 0   per (request, chunk, channel): A and B
//   pass 1   per (request, channel): over the chunks in order, the state each chunk starts from; the last into the slot
//   pass 2   per (request, chunk, channel): the chunk again, token by token from its incoming state, writing the outputs
constexpr int CHUNK = 64;

__device__ __forceinline__ void gru_gates(float zr, float xr, float bzc, float bxc, float& a, float& bb) {
    const float z = 1.0f / (1.0f + expf(-(zr + bzc)));
    const float u = xr + bxc;
    const float cand = u >= 0.f ? u + 0.5f : 1.0f / (1.0f + expf(-u));
    a = 1.0f - z; bb = z * cand;
}

template <typename TO, int PASS>
__global__ void __launch_bounds__(128)
min_gru_chunk_kernel(float* __restrict__ proj, int ld, int z_off, int x_off, int g_off, int clear_input,
                     const float* __restrict__ bz, const float* __restrict__ bx, float* __restrict__ state,
                     const int* __restrict__ q_start, const int* __restrict__ slots, int width, int max_chunks,
                     float* __restrict__ wsA, float* __restrict__ wsB, float* __restrict__ wsS,
                     TO* __restrict__ out, int out_ld, int out_off, float out_scale) {
    pdl_launch_dependents();
    const int c = blockIdx.x * 128 + threadIdx.x, b = blockIdx.z;
    if (c >= width) return;
    const float bzc = bz ? bz[c] : 0.f, bxc = bx ? bx[c] : 0.f;
    pdl_wait();
    const int t0 = q_start[b], t1 = q_start[b + 1];
    const int chunks = (t1 - t0 + CHUNK - 1) / CHUNK;
    if (PASS == 1) {
        float* sp = state + (size_t)slots[b] * width + c;
        float S = *sp;
        for (int k = 0; k < chunks; ++k) {
            const size_t at = ((size_t)b * max_chunks + k) * width + c;
            wsS[at] = S;
            S = wsA[at] * S + wsB[at];
        }
        *sp = S;
        return;
    }
    const int k = blockIdx.y;
    if (k >= chunks) return;
    const size_t at = ((size_t)b * max_chunks + k) * width + c;
    const int ta = t0 + k * CHUNK, tb = min(ta + CHUNK, t1);
    // eight tokens' inputs are fetched before any of them is used: the loads of a batch are in flight together
    constexpr int UN = 8;
    if (PASS == 0) {
        float A = 1.f, B = 0.f;
        for (int t = ta; t < tb; t += UN) {
            float zr[UN], xr[UN];
#pragma unroll
            for (int i = 0; i < UN; ++i)
                if (t + i < tb) { const float* row = proj + (size_t)(t + i) * ld; zr[i] = row[z_off + c]; xr[i] = row[x_off + c]; }
#pragma unroll
            for (int i = 0; i < UN; ++i)
                if (t + i < tb) {
                    float a, bb;
                    gru_gates(zr[i], xr[i], bzc, bxc, a, bb);
                    A *= a; B = a * B + bb;
                }
        }
        wsA[at] = A; wsB[at] = B;
    } else {
        float S = wsS[at];
        for (int t = ta; t < tb; t += UN) {
            float zr[UN], xr[UN], gr[UN];
#pragma unroll
            for (int i = 0; i < UN; ++i)
                if (t + i < tb) {
                    float* row = proj + (size_t)(t + i) * ld;
                    zr[i] = row[z_off + c]; xr[i] = row[x_off + c]; gr[i] = row[g_off + c];
                    if (clear_input) { row[z_off + c] = 0.f; row[x_off + c] = 0.f; row[g_off + c] = 0.f; }
                }
#pragma unroll
            for (int i = 0; i < UN; ++i)
                if (t + i < tb) {
                    float a, bb;
                    gru_gates(zr[i], xr[i], bzc, bxc, a, bb);
                    S = a * S + bb;
                    out[(size_t)(t + i) * out_ld + out_off + c] = from_f32<TO>(out_scale * S * (gr[i] / (1.0f + expf(-gr[i]))));
                }
        }
    }
}

}  // namespace

// Floats of workspace the chunked form needs for a step whose longest portion has max_q_len tokens.
TFF_API long long tff_min_gru_workspace(int num_requests, int max_q_len, int width) {
    return 3LL * num_requests * ((max_q_len + CHUNK - 1) / CHUNK) * width;
}

TFF_API int tff_min_gru_chunked(float* proj, int ld, int z_off, int x_off, int g_off, int clear_input, const float* bz,
                                const float* bx, float* state, int num_slots, const int* q_start, const int* slots,
                                int num_requests, int max_q_len, int width, float* workspace, void* out, int out_dt,
                                int out_ld, int out_off, float out_scale, cudaStream_t stream) {
    if (num_requests <= 0 || max_q_len <= 0) return TFF_OK;
    if (!proj || !state || !q_start || !slots || !out || !workspace || width <= 0 || num_slots <= 0) return TFF_ERR_BAD_ARGUMENT;
    const int max_chunks = (max_q_len + CHUNK - 1) / CHUNK;
    if (num_requests > 65535 || max_chunks > 65535) return TFF_ERR_UNSUPPORTED;
    float* wsA = workspace;
    float* wsB = wsA + (size_t)num_requests * max_chunks * width;
    float* wsS = wsB + (size_t)num_requests * max_chunks * width;
    dim3 grid((width + 127) / 128, max_chunks, num_requests), grid1((width + 127) / 128, 1, num_requests);
#define TFF_GRU(TO)                                                                                                      \
    do {                                                                                                                 \
        int st = tff_launch_pdl(min_gru_chunk_kernel<TO, 0>, grid, dim3(128), 0, stream, proj, ld, z_off, x_off, g_off, 0, bz, bx, \
                                state, q_start, slots, width, max_chunks, wsA, wsB, wsS, (TO*)out, out_ld, out_off, out_scale); \
        if (st != TFF_OK) return st;                                                                                     \
        st = tff_launch_pdl(min_gru_chunk_kernel<TO, 1>, grid1, dim3(128), 0, stream, proj, ld, z_off, x_off, g_off, 0, bz, bx, \
                            state, q_start, slots, width, max_chunks, wsA, wsB, wsS, (TO*)out, out_ld, out_off, out_scale); \
        if (st != TFF_OK) return st;                                                                                     \
        return tff_launch_pdl(min_gru_chunk_kernel<TO, 2>, grid, dim3(128), 0, stream, proj, ld, z_off, x_off, g_off, clear_input, \
                              bz, bx, state, q_start, slots, width, max_chunks, wsA, wsB, wsS, (TO*)out, out_ld, out_off, out_scale); \
    } while (0)
    if (out_dt == 0) TFF_GRU(float);
    TFF_GRU(bf16);
#undef TFF_GRU
}

TFF_API int tff_min_gru(float* proj, int ld, int z_off, int x_off, int g_off, int clear_input, const float* bz,
                        const float* bx, float* state, int num_slots, const int* q_start, const int* slots,
                        int num_requests, int width, void* out, int out_dt, int out_ld, int out_off, float out_scale,
                        cudaStream_t stream) {
    if (num_requests <= 0) return TFF_OK;
    if (!proj || !state || !q_start || !slots || !out || width <= 0 || num_slots <= 0) return TFF_ERR_BAD_ARGUMENT;
    if (num_requests > 65535) return TFF_ERR_UNSUPPORTED;
    dim3 grid((width + 127) / 128, num_requests);
    if (out_dt == 0)
        return tff_launch_pdl(min_gru_kernel<float>, grid, dim3(128), 0, stream, proj, ld, z_off, x_off, g_off, clear_input,
                              bz, bx, state, q_start, slots, width, (float*)out, out_ld, out_off, out_scale);
    return tff_launch_pdl(min_gru_kernel<bf16>, grid, dim3(128), 0, stream, proj, ld, z_off, x_off, g_off, clear_input,
                          bz, bx, state, q_start, slots, width, (bf16*)out, out_ld, out_off, out_scale);
}
