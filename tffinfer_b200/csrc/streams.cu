// A residual that is several streams (hyper-connections), with layer scale: one kernel does what lies
// between two sublayers.  x holds S float32 copies of the residual per token, [rows, S, W].
//
//   write (when y is given):  x'[t] = sum_s mix[s, t] x[s] + out[t] * (scale * y),  all t from the old x[s]
//   read  (when h is given):  u = sum_s in[s] x'[s];  h = u * rsqrt(mean(u^2) + eps) * w
//
// mix, out, in are float32 [S, S], [S], [S]; a null pointer stands for the identity matrix, ones, ones, so
// S = 1 with null pointers is the plain pre-norm residual with layer scale.  scale and w may be null (ones).
// One CTA per row; a thread owns columns and holds the S values of a column in registers, so the update
// is in place.  Every sum runs over s in ascending order and the row's sum of squares is reduced in an order that
// depends on W alone: a row's result does not depend on what else is in the batch.
// With row_index, CTA r works on row row_index[r] (both parts), and h is written to row r: the last
// sublayer's write and the model's final norm only ever matter at the rows whose logits are wanted.
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 8;

template <typename TO, int NT>
__global__ void __launch_bounds__(NT)
stream_step_kernel(float* __restrict__ x, int S, int W,
                   const float* __restrict__ y, const float* __restrict__ scale,
                   const float* __restrict__ mix, const float* __restrict__ outw,
                   const float* __restrict__ inw, const float* __restrict__ w, float eps,
                   const int* __restrict__ row_index, TO* __restrict__ h, float* __restrict__ total) {
    extern __shared__ float u_row[];                 // W floats: the combined row, kept between the two passes
    __shared__ float red[32];
    __shared__ float c_mix[MAX_STREAMS * MAX_STREAMS], c_out[MAX_STREAMS], c_in[MAX_STREAMS];
    pdl_launch_dependents();
    // the coefficients and the row index are older than the kernel ahead
    if (threadIdx.x < S * S) c_mix[threadIdx.x] = mix ? mix[threadIdx.x] : ((threadIdx.x / S == threadIdx.x % S) ? 1.f : 0.f);
    if (threadIdx.x < S) {
        c_out[threadIdx.x] = outw ? outw[threadIdx.x] : 1.f;
        c_in[threadIdx.x] = inw ? inw[threadIdx.x] : 1.f;
    }
    const int r = blockIdx.x;
    const int row = row_index ? row_index[r] : r;
    __syncthreads();
    pdl_wait();
    float* xr = x + (size_t)row * S * W;
    const float* yr = y ? y + (size_t)row * W : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += NT) {
        float v[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s) v[s] = s < S ? xr[(size_t)s * W + i] : 0.f;
        if (yr) {
            const float ys = scale ? yr[i] * scale[i] : yr[i];
            float n[MAX_STREAMS];
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) {
                float a = 0.f;
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s) if (s < S && t < S) a = fmaf(c_mix[s * S + t], v[s], a);
                n[t] = t < S ? fmaf(c_out[t], ys, a) : 0.f;
            }
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) if (t < S) { v[t] = n[t]; xr[(size_t)t * W + i] = n[t]; }
        }
        if (h || total) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s) if (s < S) u = fmaf(c_in[s], v[s], u);
            u_row[i] = u;
            ss = fmaf(u, u, ss);
            if (total) total[(size_t)r * W + i] = u;
        }
    }
    if (!h) return;
    ss = block_sum<NT>(ss, red);
    const float rs = rsqrtf(ss / (float)W + eps);
    TO* o = h + (size_t)r * W;
    for (int i = threadIdx.x; i < W; i += NT) {       // a thread reads back what it wrote itself
        const float g = w ? w[i] : 1.f;
        o[i] = from_f32<TO>((u_row[i] * rs) * g);
    }
}

// out[t, c, :] = E[token[t], :] * scale for c < copies: the embedding output as the start of every stream.
template <typename TW>
__global__ void embed_streams_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                     float* __restrict__ out, int hidden, int vocab, float scale, int copies) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* o = out + (size_t)t * copies * hidden;
    const bool bad = tok < 0 || tok >= vocab;            // never a wrong row: poison instead
    const TW* row = table + (size_t)(bad ? 0 : tok) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = bad ? __int_as_float(0x7fc00000) : to_f32<TW>(row[i]) * scale;
        for (int c = 0; c < copies; ++c) o[(size_t)c * hidden + i] = v;
    }
}

}  // namespace

// x [rows_total, S, W] float32 (updated in place when y is given); y [rows_total, W] float32 or null;
// h [rows, W] of the activation type or null; total [rows, W] float32 or null (the combined row itself).
TFF_API int tff_stream_step(float* x, int S, int W, const float* y, const float* scale, const float* mix,
                            const float* outw, const float* inw, const float* w, float eps, const int* row_index,
                            void* h, int h_is_bf16, float* total, int rows, cudaStream_t stream) {
    if (rows <= 0) return TFF_OK;
    if (!x || S <= 0 || W <= 0) return TFF_ERR_BAD_ARGUMENT;
    if (S > MAX_STREAMS) return TFF_ERR_UNSUPPORTED;
    const size_t smem = (size_t)W * sizeof(float);
    if (smem > 96 * 1024) return TFF_ERR_UNSUPPORTED;
#define TFF_STREAM_LAUNCH(TO, NT)                                                                              \
    do {                                                                                                       \
        auto kern = stream_step_kernel<TO, NT>;                                                                \
        if (smem > 48 * 1024) {                                                                                \
            static bool configured = false;                                                                    \
            if (!configured) {                                                                                 \
                if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess) \
                    return TFF_ERR_LAUNCH;                                                                     \
                configured = true;                                                                             \
            }                                                                                                  \
        }                                                                                                      \
        return tff_launch_pdl(kern, dim3(rows), dim3(NT), smem, stream, x, S, W, y, scale, mix, outw, inw, w,  \
                              eps, row_index, (TO*)h, total);                                                  \
    } while (0)
    if (W >= 1024) {
        if (h_is_bf16) TFF_STREAM_LAUNCH(bf16, 256);
        TFF_STREAM_LAUNCH(float, 256);
    }
    if (h_is_bf16) TFF_STREAM_LAUNCH(bf16, 64);
    TFF_STREAM_LAUNCH(float, 64);
#undef TFF_STREAM_LAUNCH
}

TFF_API int tff_embed_streams(const int* tokens, const void* table, int table_is_bf16, float* out, int num_tokens,
                              int hidden, int vocab, float scale, int copies, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (hidden <= 0 || vocab <= 0 || copies <= 0) return TFF_ERR_BAD_ARGUMENT;
    const int nt = hidden >= 1024 ? 256 : 128;
    if (table_is_bf16)
        return tff_launch_pdl(embed_streams_kernel<bf16>, dim3(num_tokens), dim3(nt), 0, stream, tokens,
                              (const bf16*)table, out, hidden, vocab, scale, copies);
    return tff_launch_pdl(embed_streams_kernel<float>, dim3(num_tokens), dim3(nt), 0, stream, tokens,
                          (const float*)table, out, hidden, vocab, scale, copies);
}
