// Attention through a cached latent: per token the cache holds one normalised latent vector c (`rank` wide)
// and one rotated key part (`dr` wide) shared by all heads; keys and values of a head are W_uk c and W_uv c.
// The kernels never build them: a head's query is taken through W_uk once (q' = W_uk^T q, `rank` wide), scores
// are q' . c + q_rot . k_rot, the weighted sum of the latents goes through W_uv at the end.  Sliding window,
// a sink in the softmax's denominator (a learned logit per head without key or value), a gate on each head's
// output.  Scores, softmax and every sum are 32-bit.
//
// A (token, head)'s result is computed the same way whatever else the step holds: keys are dealt to the warps
// by their absolute position, each warp keeps a running maximum, sum and weighted latent, and the warps are
// merged in order.
#include "api.h"
#include "common.cuh"

namespace dlmk {
namespace {

// Per token: c_q = rmsnorm(proj[off_q : off_q + q_rank]) * qn_w  -> cq_out (activation dtype, feeds a product);
// c = rmsnorm(proj[off_kv : off_kv + rank]) * kvn_w and k_rot = rotate(proj[off_kv + rank : + dr]) -> the cache row
// of the token's slot, [rank | dr].  Rotation: entry i < rot_dims / 2 pairs with i + rot_dims / 2, angle
// position * inv_freq[i] in 32-bit; entries from rot_dims on pass unchanged.
template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ proj, int ld, int off_q, int q_rank,
                                   const float* __restrict__ qn_w, int off_kv, int rank, const float* __restrict__ kvn_w,
                                   int dr, const float* __restrict__ inv_freq, int rot_dims,
                                   const int32_t* __restrict__ positions, const int32_t* __restrict__ slots, float eps,
                                   T* cq_out, T* cache, int page_size, int total_pages, int* err) {
    __shared__ float s_part[32];
    const int t = blockIdx.x;
    const float* row = proj + (long long)t * ld;
    // the query latent
    {
        float part = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) part = fmaf(row[off_q + i], row[off_q + i], part);
        const float ss = block_sum(part, s_part);
        const float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            cq_out[(long long)t * q_rank + i] = from_f32<T>((row[off_q + i] * inv) * qn_w[i]);
    }
    if (slots == nullptr) return;
    const int s = slots[t];
    if (s < 0) return;
    if (s >= total_pages * page_size) {
        if (threadIdx.x == 0) *err = 2;
        return;
    }
    T* dst = cache + (long long)s * (rank + dr);
    float part = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) part = fmaf(row[off_kv + i], row[off_kv + i], part);
    const float ss = block_sum(part, s_part);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<T>((row[off_kv + i] * inv) * kvn_w[i]);
    const float* kr = row + off_kv + rank;
    const int half = rot_dims / 2;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < dr; i += blockDim.x) {
        float v;
        if (i < half) {
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            v = kr[i] * cs - kr[i + half] * sn;
        } else if (i < 2 * half) {
            float sn, cs;
            sincosf(pos * inv_freq[i - half], &sn, &cs);
            v = kr[i] * cs + kr[i - half] * sn;
        } else {
            v = kr[i];
        }
        dst[rank + i] = from_f32<T>(v);
    }
}

constexpr int LAT_WARPS = 4;

// One block a (token, head).  NC: latent entries a lane keeps (rank <= 32 NC).
template <typename T, int NC>
__global__ void latent_attention_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ gate, int ldg,
                                        const T* __restrict__ w_uk, const T* __restrict__ w_uv,
                                        const float* __restrict__ sink, const T* __restrict__ cache,
                                        const int32_t* __restrict__ block_table, int table_width,
                                        const int32_t* __restrict__ token_req, const int32_t* __restrict__ positions,
                                        const float* __restrict__ inv_freq, int rot_dims, T* out, int H, int dn, int dr,
                                        int dv, int rank, int page_size, int total_pages, int window, float scale,
                                        int* err) {
    extern __shared__ float sm[];
    float* s_qn = sm;                         // [dn]   unrotated query part
    float* s_qr = s_qn + dn;                  // [dr]   rotated query part
    float* s_qa = s_qr + dr;                  // [rank] query taken through W_uk
    float* s_acc = s_qa + rank;               // [LAT_WARPS][rank]
    float* s_ml = s_acc + LAT_WARPS * rank;   // [LAT_WARPS][2]
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = positions[t];
    const float* qrow = q + (long long)t * ldq + (long long)h * (dn + dr);
    for (int i = threadIdx.x; i < dn; i += blockDim.x) s_qn[i] = qrow[i];
    {
        const float* qr = qrow + dn;
        const int half = rot_dims / 2;
        const float pos = (float)p;
        for (int i = threadIdx.x; i < dr; i += blockDim.x) {
            float v;
            if (i < half) {
                float sn, cs;
                sincosf(pos * inv_freq[i], &sn, &cs);
                v = qr[i] * cs - qr[i + half] * sn;
            } else if (i < 2 * half) {
                float sn, cs;
                sincosf(pos * inv_freq[i - half], &sn, &cs);
                v = qr[i] * cs + qr[i - half] * sn;
            } else {
                v = qr[i];
            }
            s_qr[i] = v;
        }
    }
    __syncthreads();
    for (int r = threadIdx.x; r < rank; r += blockDim.x) {
        const T* wc = w_uk + (long long)h * dn * rank + r;
        float acc = 0.f;
        for (int d = 0; d < dn; ++d) acc = fmaf(s_qn[d], to_f32(wc[(long long)d * rank]), acc);
        s_qa[r] = acc;
    }
    __syncthreads();

    const int req = token_req[t];
    const int32_t* table = block_table + (long long)req * table_width;
    const int lo = window > 0 ? (p - window + 1 > 0 ? p - window + 1 : 0) : 0;
    const int width = rank + dr;
    float m = -INFINITY, l = 0.f;
    float acc[NC];
#pragma unroll
    for (int n = 0; n < NC; ++n) acc[n] = 0.f;
    // key j belongs to warp j mod LAT_WARPS
    int j = lo + ((warp - lo) % LAT_WARPS + LAT_WARPS) % LAT_WARPS;
    for (; j <= p; j += LAT_WARPS) {
        const int lp = j / page_size;
        const int page = lp < table_width ? table[lp] : -1;
        if (page < 0 || page >= total_pages) {
            if (lane == 0) *err = 3;
            continue;
        }
        const T* row = cache + ((long long)page * page_size + (j - lp * page_size)) * width;
        float c[NC];
        float dot = 0.f;
#pragma unroll
        for (int n = 0; n < NC; ++n) {
            const int r = lane + 32 * n;
            c[n] = r < rank ? to_f32(row[r]) : 0.f;
            if (r < rank) dot = fmaf(s_qa[r], c[n], dot);
        }
        for (int i = lane; i < dr; i += 32) dot = fmaf(s_qr[i], to_f32(row[rank + i]), dot);
        const float sc = warp_sum(dot) * scale;
        const float m_new = fmaxf(m, sc);
        const float corr = expf(m - m_new);          // m = -inf at the first key: 0
        const float pw = expf(sc - m_new);
        l = l * corr + pw;
#pragma unroll
        for (int n = 0; n < NC; ++n) acc[n] = fmaf(pw, c[n], acc[n] * corr);
        m = m_new;
    }
#pragma unroll
    for (int n = 0; n < NC; ++n) {
        const int r = lane + 32 * n;
        if (r < rank) s_acc[warp * rank + r] = acc[n];
    }
    if (lane == 0) {
        s_ml[2 * warp] = m;
        s_ml[2 * warp + 1] = l;
    }
    __syncthreads();
    // merge: the sink takes part in the maximum and in the denominator, not in the sum of values
    const float snk = sink ? sink[h] : -INFINITY;
    float mm = snk;
#pragma unroll
    for (int w = 0; w < LAT_WARPS; ++w) mm = fmaxf(mm, s_ml[2 * w]);
    float f[LAT_WARPS];
    float den = sink ? expf(snk - mm) : 0.f;
#pragma unroll
    for (int w = 0; w < LAT_WARPS; ++w) {
        f[w] = s_ml[2 * w + 1] > 0.f ? expf(s_ml[2 * w] - mm) : 0.f;
        den += s_ml[2 * w + 1] * f[w];
    }
    const float inv = den > 0.f ? 1.0f / den : 0.f;
    __syncthreads();
    for (int r = threadIdx.x; r < rank; r += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < LAT_WARPS; ++w) v = fmaf(s_acc[w * rank + r], f[w], v);
        s_qa[r] = v * inv;                           // the weighted latent (s_qa is free now)
    }
    __syncthreads();
    const float gt = gate ? 1.0f / (1.0f + expf(-gate[(long long)t * ldg + h])) : 1.0f;
    for (int d = warp; d < dv; d += LAT_WARPS) {
        const T* wr = w_uv + ((long long)h * dv + d) * rank;
        float a = 0.f;
        for (int r = lane; r < rank; r += 32) a = fmaf(to_f32(wr[r]), s_qa[r], a);
        a = warp_sum(a);
        if (lane == 0) out[(long long)t * H * dv + (long long)h * dv + d] = from_f32<T>(a * gt);
    }
}

}  // namespace

void latent_prep(const float* proj, int ld, int off_q, int q_rank, const float* qn_w, int off_kv, int rank,
                 const float* kvn_w, int dr, const float* inv_freq, int rot_dims, const int32_t* positions,
                 const int32_t* slots, float eps, void* cq_out, void* cache, int page_size, int total_pages, int T,
                 int dtype, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(rot_dims % 2 == 0 && rot_dims >= 0 && rot_dims <= dr, "latent_prep: rotated dims must be even and <= dr");
    int* err = error_flag_ptr();
    if (dtype == F32)
        latent_prep_kernel<float><<<T, 128, 0, stream>>>(proj, ld, off_q, q_rank, qn_w, off_kv, rank, kvn_w, dr, inv_freq,
                                                        rot_dims, positions, slots, eps, static_cast<float*>(cq_out),
                                                        static_cast<float*>(cache), page_size, total_pages, err);
    else
        latent_prep_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>(
            proj, ld, off_q, q_rank, qn_w, off_kv, rank, kvn_w, dr, inv_freq, rot_dims, positions, slots, eps,
            static_cast<__nv_bfloat16*>(cq_out), static_cast<__nv_bfloat16*>(cache), page_size, total_pages, err);
    check_launch("latent_prep");
}

namespace {
template <typename T, int NC>
void launch_latent(const float* q, int ldq, const float* gate, int ldg, const void* w_uk, const void* w_uv,
                   const float* sink, const void* cache, const int32_t* block_table, int table_width,
                   const int32_t* token_req, const int32_t* positions, const float* inv_freq, int rot_dims, void* out,
                   int Tn, int H, int dn, int dr, int dv, int rank, int page_size, int total_pages, int window,
                   float scale, cudaStream_t stream) {
    const size_t smem = ((size_t)dn + dr + rank + (size_t)LAT_WARPS * rank + 2 * LAT_WARPS) * sizeof(float);
    DLM_CHECK(smem <= 200 * 1024, "latent_attention: sizes too large for shared memory");
    auto kern = latent_attention_kernel<T, NC>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<dim3(Tn, H), 32 * LAT_WARPS, smem, stream>>>(
        q, ldq, gate, ldg, static_cast<const T*>(w_uk), static_cast<const T*>(w_uv), sink, static_cast<const T*>(cache),
        block_table, table_width, token_req, positions, inv_freq, rot_dims, static_cast<T*>(out), H, dn, dr, dv, rank,
        page_size, total_pages, window, scale, error_flag_ptr());
    check_launch("latent_attention");
}
}  // namespace

void latent_attention(const float* q, int ldq, const float* gate, int ldg, const void* w_uk, const void* w_uv,
                      const float* sink, const void* cache, const int32_t* block_table, int table_width,
                      const int32_t* token_req, const int32_t* positions, const float* inv_freq, int rot_dims, void* out,
                      int T, int H, int dn, int dr, int dv, int rank, int page_size, int total_pages, int window,
                      float scale, int dtype, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(rank >= 1 && rank <= 1024, "latent_attention: latent size 1..1024");
    DLM_CHECK(rot_dims % 2 == 0 && rot_dims <= dr, "latent_attention: rotated dims must be even and <= dr");
#define DLM_LAT(TT, NC)                                                                                              \
    launch_latent<TT, NC>(q, ldq, gate, ldg, w_uk, w_uv, sink, cache, block_table, table_width, token_req, positions, \
                          inv_freq, rot_dims, out, T, H, dn, dr, dv, rank, page_size, total_pages, window, scale, stream)
    const int nc = (rank + 31) / 32;
    if (dtype == F32) {
        if (nc <= 4) DLM_LAT(float, 4);
        else if (nc <= 8) DLM_LAT(float, 8);
        else if (nc <= 16) DLM_LAT(float, 16);
        else DLM_LAT(float, 32);
    } else {
        if (nc <= 4) DLM_LAT(__nv_bfloat16, 4);
        else if (nc <= 8) DLM_LAT(__nv_bfloat16, 8);
        else if (nc <= 16) DLM_LAT(__nv_bfloat16, 16);
        else DLM_LAT(__nv_bfloat16, 32);
    }
#undef DLM_LAT
}

}  // namespace dlmk
