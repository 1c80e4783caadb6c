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

}  // namespace

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
