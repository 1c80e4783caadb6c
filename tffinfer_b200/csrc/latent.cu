// What lies between the projections of a latent attention and its token mixing.
//
// latent_finish, one block per token, on the float32 accumulators of the merged down-projection
//   row t = [ q latent (q_rank) | kv latent (kv_rank) | shared key part (rot_dim) ]:
// * cq[t] = rmsnorm(q latent) * wq                         -> the up-projection's input rows
// * c[t]  = rmsnorm(kv latent) * wkv                       -> elements 0 .. kv_rank-1 of the token's cache slot
// * r[t]  = the shared key part, its first rot_dims elements turned pair by pair (2i, 2i+1) by the angle
//   float(position) * freq[i]                              -> elements kv_rank .. kv_rank+rot_dim-1 of the slot
//   (a cache of ONE plane: a token's slot holds [c | r]; kv_rank = 0 or no cache: a layer that reads another layer's)
// rmsnorm(x) = x * rsqrt(mean(x^2) + eps), then times the weight; all float32, only the stores round.
//
// latent_q_rot, one warp per (token, head): the rotated part of a query head, q[t, h*(dim+rot_dim) + dim ..] (the
// up-projection's output in the activation type; the rotation itself is float32), turned
// the same way, into columns kv_rank .. of the head's row of the absorbed query [T, heads*(kv_rank+rot_dim)].
#include "common.cuh"

namespace {

template <typename TQ, typename TC>
__global__ void __launch_bounds__(128)
latent_finish_kernel(float* __restrict__ proj, int ld, int clear_input, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                     const float* __restrict__ wq, const float* __restrict__ wkv, float eps, const float* __restrict__ freq,
                     const int* __restrict__ positions, const int* __restrict__ tok_req,
                     const int* __restrict__ block_table, int table_width, TC* __restrict__ cache, long long page_stride,
                     int page_size, int slot_elems, TQ* __restrict__ cq, TC* __restrict__ dense_out) {
    __shared__ float red[32];
    pdl_launch_dependents();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int pos = positions[t];
    pdl_wait();
    float* row = proj + (size_t)t * ld;
    if (q_rank > 0) {
        float ss = 0.f;
        for (int i = tid; i < q_rank; i += 128) { const float x = row[i]; ss = fmaf(x, x, ss); }
        ss = block_sum<128>(ss, red);
        const float r = rsqrtf(ss / (float)q_rank + eps);
        for (int i = tid; i < q_rank; i += 128) {
            const float x = row[i];
            if (clear_input) row[i] = 0.f;
            cq[(size_t)t * q_rank + i] = from_f32<TQ>((x * r) * wq[i]);
        }
    }
    if (cache == nullptr || kv_rank <= 0) return;
    const int page = block_table[(size_t)tok_req[t] * table_width + pos / page_size];
    if (page < 0) return;                                        // no page: the host never schedules this
    TC* slot = cache + (size_t)page * page_stride + (size_t)(pos % page_size) * slot_elems;
    TC* drow = dense_out ? dense_out + (size_t)t * (kv_rank + rot_dim) : nullptr;   // the same vector in a plain row
    float* src = row + q_rank;
    float ss = 0.f;
    for (int i = tid; i < kv_rank; i += 128) { const float x = src[i]; ss = fmaf(x, x, ss); }
    ss = block_sum<128>(ss, red);
    const float r = rsqrtf(ss / (float)kv_rank + eps);
    for (int i = tid; i < kv_rank; i += 128) {
        const float x = src[i];
        if (clear_input) src[i] = 0.f;
        slot[i] = from_f32<TC>((x * r) * wkv[i]);
        if (drow) drow[i] = slot[i];
    }
    float* rs = src + kv_rank;
    TC* rd = slot + kv_rank;
    const int half = rot_dims >> 1;
    for (int i = tid; i < half; i += 128) {
        const float u = rs[2 * i], v = rs[2 * i + 1];
        if (clear_input) { rs[2 * i] = 0.f; rs[2 * i + 1] = 0.f; }
        float s, c;
        sincosf((float)pos * freq[i], &s, &c);
        rd[2 * i] = from_f32<TC>(u * c - v * s);
        rd[2 * i + 1] = from_f32<TC>(v * c + u * s);
        if (drow) { drow[kv_rank + 2 * i] = rd[2 * i]; drow[kv_rank + 2 * i + 1] = rd[2 * i + 1]; }
    }
    for (int i = 2 * half + tid; i < rot_dim; i += 128) {
        const float x = rs[i];
        if (clear_input) rs[i] = 0.f;
        rd[i] = from_f32<TC>(x);
        if (drow) drow[kv_rank + i] = rd[i];
    }
}

// keys[t, h, dim .. dim + rot_dim) = latent[t, kv_rank .. kv_rank + rot_dim): the shared rotated key part into every head's
// key row, for the form of the attention that makes per-head keys (one warp per (token, head))
template <typename T>
__global__ void __launch_bounds__(128)
latent_spread_kernel(const T* __restrict__ latent, int kv_rank, int rot_dim, T* __restrict__ keys, int dim, int heads,
                     int num_tokens) {
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)num_tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item % heads);
    pdl_wait();
    const T* src = latent + (size_t)t * (kv_rank + rot_dim) + kv_rank;
    T* dst = keys + ((size_t)t * heads + h) * (dim + rot_dim) + dim;
    for (int i = lane; i < rot_dim; i += 32) dst[i] = src[i];
}

template <typename TQ>
__global__ void __launch_bounds__(128)
latent_q_rot_kernel(const TQ* q, int dim, int rot_dim, int rot_dims, const float* __restrict__ freq,
                    const int* __restrict__ positions, TQ* q_lat, int kv_rank, int heads, int num_tokens) {
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)num_tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item % heads);
    const int pos = positions[t];
    pdl_wait();
    const TQ* src = q + ((size_t)t * heads + h) * (dim + rot_dim) + dim;
    TQ* dst = q_lat + ((size_t)t * heads + h) * (kv_rank + rot_dim) + kv_rank;
    const int half = rot_dims >> 1;
    for (int i = lane; i < half; i += 32) {
        const float u = to_f32<TQ>(src[2 * i]), v = to_f32<TQ>(src[2 * i + 1]);
        float s, c;
        sincosf((float)pos * freq[i], &s, &c);
        dst[2 * i] = from_f32<TQ>(u * c - v * s);
        dst[2 * i + 1] = from_f32<TQ>(v * c + u * s);
    }
    for (int i = 2 * half + lane; i < rot_dim; i += 32) dst[i] = src[i];
}

}  // namespace

// is_bf16: cq and the cache are bfloat16, else float32.  ``cache`` is the start of the layer's share of a one-plane,
// one-head pool whose pages are page_stride elements apart; null (or kv_rank 0) when the layer keeps no cache.
TFF_API int tff_latent_finish(float* proj, int ld, int clear_input, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                              const float* wq, const float* wkv, float eps, const float* freq, const int* positions,
                              const int* tok_req, const int* block_table, int table_width, void* cache,
                              long long page_stride, int page_size, int slot_elems, void* cq, int is_bf16,
                              void* dense_out, int num_tokens, cudaStream_t stream) {
    if (num_tokens <= 0) return TFF_OK;
    if (!proj || q_rank < 0 || kv_rank < 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1))
        return TFF_ERR_BAD_ARGUMENT;
    if (q_rank > 0 && (!cq || !wq)) return TFF_ERR_BAD_ARGUMENT;
    if (cache && kv_rank > 0 && (!wkv || !block_table || page_size <= 0 || slot_elems < kv_rank + rot_dim || (rot_dims > 0 && !freq)))
        return TFF_ERR_BAD_ARGUMENT;
    if (is_bf16)
        return tff_launch_pdl(latent_finish_kernel<bf16, bf16>, dim3(num_tokens), dim3(128), 0, stream, proj, ld, clear_input,
                              q_rank, kv_rank, rot_dim, rot_dims, wq, wkv, eps, freq, positions, tok_req, block_table,
                              table_width, (bf16*)cache, page_stride, page_size, slot_elems, (bf16*)cq, (bf16*)dense_out);
    return tff_launch_pdl(latent_finish_kernel<float, float>, dim3(num_tokens), dim3(128), 0, stream, proj, ld, clear_input,
                          q_rank, kv_rank, rot_dim, rot_dims, wq, wkv, eps, freq, positions, tok_req, block_table,
                          table_width, (float*)cache, page_stride, page_size, slot_elems, (float*)cq, (float*)dense_out);
}

TFF_API int tff_latent_q_rot(const void* q, int dim, int rot_dim, int rot_dims, const float* freq, const int* positions,
                             void* q_lat, int is_bf16, int kv_rank, int heads, int num_tokens, cudaStream_t stream) {
    if (num_tokens <= 0 || rot_dim <= 0) return TFF_OK;
    if (!q || !q_lat || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1) || (rot_dims > 0 && !freq)) return TFF_ERR_BAD_ARGUMENT;
    const long long items = (long long)num_tokens * heads;
    dim3 grid((unsigned)((items + 3) / 4));
    if (is_bf16)
        return tff_launch_pdl(latent_q_rot_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)q, dim, rot_dim, rot_dims, freq, positions,
                              (bf16*)q_lat, kv_rank, heads, num_tokens);
    return tff_launch_pdl(latent_q_rot_kernel<float>, grid, dim3(128), 0, stream, (const float*)q, dim, rot_dim, rot_dims, freq, positions,
                          (float*)q_lat, kv_rank, heads, num_tokens);
}

TFF_API int tff_latent_spread(const void* latent, int kv_rank, int rot_dim, void* keys, int dim, int heads, int is_bf16,
                              int num_tokens, cudaStream_t stream) {
    if (num_tokens <= 0 || rot_dim <= 0) return TFF_OK;
    if (!latent || !keys || kv_rank < 0 || dim < 0 || heads <= 0) return TFF_ERR_BAD_ARGUMENT;
    const long long items = (long long)num_tokens * heads;
    dim3 grid((unsigned)((items + 3) / 4));
    if (is_bf16)
        return tff_launch_pdl(latent_spread_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)latent, kv_rank, rot_dim,
                              (bf16*)keys, dim, heads, num_tokens);
    return tff_launch_pdl(latent_spread_kernel<float>, grid, dim3(128), 0, stream, (const float*)latent, kv_rank, rot_dim,
                          (float*)keys, dim, heads, num_tokens);
}
