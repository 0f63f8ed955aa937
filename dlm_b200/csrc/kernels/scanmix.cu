// Kernels of mixers that run side by side and of the diagonal state-space scan:
//   * selective_scan: S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n, y_c = S[c, :] . C + D_c x_c, with the
//     step size dt_c = softplus(raw + bias) per channel and token, and the gate y silu(z) applied on the way out;
//   * qk_norm_write: RMS norm over the whole query and the whole key projection, a query temperature that grows
//     with the position, and the write of queries, keys and values in the layout of the attention kernels;
//   * rotate_heads: rotary positions applied in place to 32-bit rows (two runs of heads, each with a factor);
//   * branch_norm_add: resid += coef * sum_b rms_norm(branch_b) * w_b for one or two branch outputs;
//   * rmsnorm_pair: two RMS norms of the same rows (one statistic, two weights);
//   * concat_rows: [a | b] in the activation dtype (the input of a product that reads two residuals).
//
// Everything is computed in 32-bit whatever the activation dtype is; only what a kernel hands to a matrix product
// or to the cache is rounded.  A token's result depends on the tokens before it in its own request only, in an
// order that does not depend on how the request was cut into steps.
#include "api.h"
#include "common.cuh"

namespace dlmk {
namespace {

__device__ __forceinline__ float softplus_f(float z) { return z > 30.0f ? z : log1pf(expf(z)); }

__device__ __forceinline__ void copy4_async(float* dst_smem, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copy16_async(float* dst_smem, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src)
                 : "memory");
}
template <int N> __device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ------------------------------------------------------------------ selective scan
// A block owns (a run of `chans` channels, a request).  A channel's N states are shared by `parts` neighbouring
// lanes, lane `part` keeps states part, part + parts, ... in registers (NPT of them).  Tokens come in tiles of TILE
// by asynchronous copies into a ring of buffers, three tiles ahead: per token B and C (N each, shared by all channels), and the
// block's x, raw dt and z.  A tile is worked on in three phases: (1) all threads turn its raw step sizes into
// dt = softplus(raw + bias) at once; (2) every lane walks the tile's tokens with its own states and leaves its part
// of each token's sum over states in shared memory: a token's only dependence on the one before it is the state's
// own multiply-add, so a full tile's walk is unrolled; (3) all threads add the parts of a (token, channel) in lane
// order, add D x, apply the gate and store.  The decay exp(dt A) is 2^(dt A log2 e) with A log2 e kept in registers.
constexpr int SCAN_THREADS = 128;
constexpr int SCAN_TILE = 32;
constexpr int SCAN_STAGES = 4;     // tiles asked for ahead of the one worked on: a tile's walk is shorter than a trip to memory

template <int NPT, typename TOut>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ dt_raw, int lddt,
                      const float* __restrict__ bc, int ldbc, const float* __restrict__ z, int ldz,
                      const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ D,
                      float* state, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ state_slot, TOut* out,
                      int ldo, int inner, int N, int parts, int wide) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    extern __shared__ __align__(16) float sm[];       // [STAGES][TILE][2 N + 3 chans]: B, C, x, dt, z;  then [TILE][chans][parts + 1]
    const int chans = SCAN_THREADS / parts;
    const int part = threadIdx.x % parts, col = threadIdx.x / parts;
    const int c0 = blockIdx.x * chans, c = c0 + col;
    const int r = blockIdx.y;
    const bool live = c < inner;
    const int rl = 2 * N + 3 * chans;
    // a channel's parts lie side by side, channels parts + 1 apart: lanes that add up different channels' parts read
    // different banks
    float* ps = sm + SCAN_STAGES * (size_t)SCAN_TILE * rl;
    const int ps_ld = chans * (parts + 1);
    float* mine = ps + col * (parts + 1) + part;
    float* st = state + ((long long)state_slot[r] * inner + (live ? c : 0)) * N;
    float s[NPT], a2[NPT];
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = part + parts * i;
        const bool ok = live && n < N;
        s[i] = ok ? st[n] : 0.f;
        a2[i] = ok ? -expf(A_log[(long long)c * N + n]) * 1.4426950408889634f : 0.f;
    }
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    const int n_tiles = (t1 - t0 + SCAN_TILE - 1) / SCAN_TILE;
    const int nch = min(chans, inner - c0);
    // `wide`: every run of a token's inputs starts on a 16-byte boundary and is a multiple of four floats
    auto fetch = [&](int k) {             // (a tile beyond the last: an empty group, so that the count of groups holds)
        float* buf = sm + (size_t)(k % SCAN_STAGES) * SCAN_TILE * rl;
        const int first = t0 + k * SCAN_TILE, n = min(SCAN_TILE, t1 - first);
        const int lane = threadIdx.x & 31, nwarp = SCAN_THREADS >> 5;
        for (int tok = threadIdx.x >> 5; tok < n; tok += nwarp) {
            const long long t = first + tok;
            const float* src_bc = bc + t * ldbc;
            const float* src_x = x + t * ldx + c0;
            const float* src_dt = dt_raw + t * lddt + c0;
            const float* src_z = z + t * ldz + c0;
            float* dst = buf + (size_t)tok * rl;
            if (wide) {
                for (int i = 4 * lane; i < 2 * N; i += 128) copy16_async(dst + i, src_bc + i);
                for (int i = 4 * lane; i < nch; i += 128) {
                    copy16_async(dst + 2 * N + i, src_x + i);
                    copy16_async(dst + 2 * N + chans + i, src_dt + i);
                    copy16_async(dst + 2 * N + 2 * chans + i, src_z + i);
                }
            } else {
                for (int i = lane; i < 2 * N; i += 32) copy4_async(dst + i, src_bc + i);
                for (int i = lane; i < nch; i += 32) {
                    copy4_async(dst + 2 * N + i, src_x + i);
                    copy4_async(dst + 2 * N + chans + i, src_dt + i);
                    copy4_async(dst + 2 * N + 2 * chans + i, src_z + i);
                }
            }
        }
        copies_commit();
    };
    // one token of the walk: the lane's states move on, its part of the token's sum goes to shared memory
    auto one = [&](const float* row, float* dst) {
        const float dt = row[2 * N + chans + col];
        const float dx = dt * row[2 * N + col];
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int n_i = part + parts * i;
            if (n_i < N) {
                s[i] = fmaf(exp2f(dt * a2[i]), s[i], dx * row[n_i]);
                sum = fmaf(s[i], row[N + n_i], sum);
            }
        }
        *dst = sum;
    };
    for (int k = 0; k < SCAN_STAGES - 1; ++k) fetch(k);
    for (int k = 0; k < n_tiles; ++k) {
        fetch(k + SCAN_STAGES - 1);          // into the buffer of tile k - 1, which the barrier below the last phase freed
        copies_wait<SCAN_STAGES - 1>();
        __syncthreads();
        float* buf = sm + (size_t)(k % SCAN_STAGES) * SCAN_TILE * rl;
        const int first = t0 + k * SCAN_TILE, n = min(SCAN_TILE, t1 - first);
        for (int idx = threadIdx.x; idx < n * nch; idx += SCAN_THREADS) {
            const int tok = idx / nch, ch = idx - tok * nch;
            float* p = buf + (size_t)tok * rl + 2 * N + chans + ch;
            *p = softplus_f(*p + dt_bias[c0 + ch]);
        }
        __syncthreads();
        if (live) {
            if (n == SCAN_TILE) {
#pragma unroll
                for (int tok = 0; tok < SCAN_TILE; ++tok) one(buf + (size_t)tok * rl, mine + tok * ps_ld);
            } else {
                for (int tok = 0; tok < n; ++tok) one(buf + (size_t)tok * rl, mine + tok * ps_ld);
            }
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < n * nch; idx += SCAN_THREADS) {
            const int tok = idx / nch, ch = idx - tok * nch;
            const float* row = buf + (size_t)tok * rl;
            const float* pp = ps + tok * ps_ld + ch * (parts + 1);
            float v = 0.f;
            for (int p = 0; p < parts; ++p) v += pp[p];
            const float y = fmaf(D[c0 + ch], row[2 * N + ch], v);
            out[(long long)(first + tok) * ldo + c0 + ch] = from_f32<TOut>(y * silu_f(row[2 * N + 2 * chans + ch]));
        }
        __syncthreads();                     // this tile's buffer and the sums may be written again
    }
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = part + parts * i;
        if (live && n < N) st[n] = s[i];
    }
}

// ------------------------------------------------- whole-projection norms, temperature, cache write
// One block a token.  qkv f32 row: [q: nh * d | k: nkv * d | v: nkv * dv].  q and k are each divided by the root
// mean square of the WHOLE projection (all heads at once) and multiplied by a weight per entry; q also by the
// temperature 1 + coef * ln(floor((p + 1) / every) + 1) of its position p (every == 0: none).  Heads are written
// D wide (D >= d, dv; entries beyond a head's own size are zero) so that keys and values share one head size.
template <typename T>
__global__ void qk_norm_write_kernel(const float* qkv, int ld, const int32_t* __restrict__ positions,
                                     const float* __restrict__ qn_w, const float* __restrict__ kn_w, float eps,
                                     float temp_coef, int temp_every, const int32_t* __restrict__ slots, T* q_out,
                                     T* k_cache, T* v_cache, int nh, int nkv, int d, int dv, int D, int page_size,
                                     int total_pages, int* err) {
    __shared__ float s_part[32];
    dep_wait();
    dep_launch_next();
    const int t = blockIdx.x;
    const int Q = nh * d, K = nkv * d, V = nkv * dv;
    const float* row = qkv + (long long)t * ld;
    int in_page = 0, page = -1;
    if (slots != nullptr) {
        const int s = slots[t];
        if (s >= 0) {
            page = s / page_size;
            in_page = s % page_size;
            if (page >= total_pages) {
                if (threadIdx.x == 0) *err = 2;
                page = -1;
            }
        }
    }
    float pq = 0.f, pk = 0.f;
    for (int i = threadIdx.x; i < Q; i += blockDim.x) pq = fmaf(row[i], row[i], pq);
    for (int i = threadIdx.x; i < K; i += blockDim.x) pk = fmaf(row[Q + i], row[Q + i], pk);
    const float sq = block_sum(pq, s_part);
    const float sk = block_sum(pk, s_part);
    float fq = qn_w != nullptr ? 1.0f / sqrtf(sq / (float)Q + eps) : 1.0f;
    const float fk = kn_w != nullptr ? 1.0f / sqrtf(sk / (float)K + eps) : 1.0f;
    float temp = 1.0f;
    if (temp_every > 0) temp = 1.0f + temp_coef * logf((float)((positions[t] + 1) / temp_every) + 1.0f);
    for (int idx = threadIdx.x; idx < nh * D; idx += blockDim.x) {
        const int h = idx / D, i = idx - h * D;
        float v = 0.f;
        if (i < d) {
            const int e = h * d + i;
            v = (row[e] * fq) * (qn_w != nullptr ? qn_w[e] : 1.0f) * temp;
        }
        q_out[(long long)t * nh * D + idx] = from_f32<T>(v);
    }
    if (page >= 0) {
        for (int idx = threadIdx.x; idx < nkv * D; idx += blockDim.x) {
            const int h = idx / D, i = idx - h * D;
            float kv = 0.f, vv = 0.f;
            if (i < d) {
                const int e = h * d + i;
                kv = (row[Q + e] * fk) * (kn_w != nullptr ? kn_w[e] : 1.0f);
            }
            if (i < dv) vv = row[Q + K + h * dv + i];
            const long long o = (((long long)page * nkv + h) * page_size + in_page) * D + i;
            k_cache[o] = from_f32<T>(kv);
            v_cache[o] = from_f32<T>(vv);
        }
    }
    (void)V;
}

// ------------------------------------------------------------------ rotation in place
// One block a token.  x f32 rows; two runs of `heads` heads of `dim` entries start at columns off_a and off_b.
// In every head the first rot_dims entries are rotated (entry i with entry i + rot_dims / 2, angle
// position * inv_freq[i]); then the whole head is multiplied by the run's factor.
__global__ void rotate_heads_kernel(float* x, int ld, const int32_t* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int rot_dims, int heads, int dim, int off_a,
                                    float scale_a, int off_b, float scale_b) {
    extern __shared__ float sc[];                  // [2][rot_dims / 2]: sines, cosines
    const int t = blockIdx.x;
    const int half = rot_dims / 2;
    const float pos = (float)positions[t];         // (positions and frequencies are the step's inputs)
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        sc[i] = sn;
        sc[half + i] = cs;
    }
    dep_wait();
    dep_launch_next();
    __syncthreads();
    float* row = x + (long long)t * ld;
    const int per = heads * dim;
    for (int idx = threadIdx.x; idx < 2 * per; idx += blockDim.x) {
        const int run = idx / per, e = idx - run * per;
        const int h = e / dim, i = e - h * dim;
        float* head = row + (run ? off_b : off_a) + h * dim;
        const float f = run ? scale_b : scale_a;
        if (i < half) {
            const float u = head[i], v = head[i + half];
            const float sn = sc[i], cs = sc[half + i];
            head[i] = (u * cs - v * sn) * f;
            head[i + half] = (v * cs + u * sn) * f;
        } else if (i >= 2 * half && f != 1.0f) {
            head[i] *= f;
        }
    }
}

// --------------------------------------------------------- sum of normed branch outputs
// One block a token: resid[t] += coef * (a / rms(a) * wa + b / rms(b) * wb)   (b == nullptr: one branch).
__global__ void branch_norm_add_kernel(float* resid, const float* a, const float* __restrict__ wa, const float* b,
                                       const float* __restrict__ wb, float eps, float coef, int H) {
    __shared__ float s_part[32];
    dep_wait();
    dep_launch_next();
    const long long t = blockIdx.x;
    const float* ar = a + t * H;
    const float* br = b != nullptr ? b + t * H : nullptr;
    float pa = 0.f, pb = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        pa = fmaf(ar[i], ar[i], pa);
        if (br != nullptr) pb = fmaf(br[i], br[i], pb);
    }
    const float sa = block_sum(pa, s_part);
    const float sb = block_sum(pb, s_part);
    const float fa = 1.0f / sqrtf(sa / (float)H + eps), fb = 1.0f / sqrtf(sb / (float)H + eps);
    float* o = resid + t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = (ar[i] * fa) * wa[i];
        if (br != nullptr) v += (br[i] * fb) * wb[i];
        o[i] += coef * v;
    }
}

// ------------------------------------------------------------ two norms of the same rows
// One block a row: out_a = x / rms(x) * wa, out_b = x / rms(x) * wb (one statistic, two weights).
template <typename T>
__global__ void rmsnorm_pair_kernel(const float* x, const float* __restrict__ wa, const float* __restrict__ wb, T* out_a,
                                    T* out_b, int H, float eps) {
    __shared__ float s_part[32];
    dep_wait();
    dep_launch_next();
    const long long t = blockIdx.x;
    const float* row = x + t * H;
    float part = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) part = fmaf(row[i], row[i], part);
    const float inv = 1.0f / sqrtf(block_sum(part, s_part) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = row[i] * inv;
        out_a[t * H + i] = from_f32<T>(v * wa[i]);
        out_b[t * H + i] = from_f32<T>(v * wb[i]);
    }
}

// ------------------------------------------------------------------ two rows side by side
template <typename T>
__global__ void concat_rows_kernel(const float* a, const float* b, T* out, int H) {
    dep_wait();
    dep_launch_next();
    const long long t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        out[t * 2 * H + i] = from_f32<T>(a[t * H + i]);
        out[t * 2 * H + H + i] = from_f32<T>(b[t * H + i]);
    }
}

}  // namespace

void selective_scan(const float* x, int ldx, const float* dt_raw, int lddt, const float* bc, int ldbc, const float* z,
                    int ldz, const float* dt_bias, const float* A_log, const float* D, float* state,
                    const int32_t* cu_q, const int32_t* state_slot, void* out, int ldo, int R, int inner, int N,
                    int out_dtype, cudaStream_t stream) {
    if (R <= 0 || inner <= 0) return;
    DLM_CHECK(N >= 1 && N <= 256, "selective_scan: state size 1..256");
    // few states a lane, so that a channel spreads over lanes; fewer still while the launch would not fill the
    // machine three times over (a prompt of one request is walked by inner / chans blocks).  Measured on a prompt of
    // 2,048 tokens, 4,096 channels of 16 states: 2 / 4 / 8 / 16 lanes a channel take 1,446 / 789 / 597 / 495 us: the
    // walk is a chain of dependent steps per lane, and what shortens a lane's chain shortens the kernel
    int parts = 1;
    while (parts < 32 && (N + parts - 1) / parts > 4) parts <<= 1;
    while (parts < 32 && (N + parts - 1) / parts > 1 &&
           (long long)((inner + SCAN_THREADS / parts - 1) / (SCAN_THREADS / parts)) * R < 3LL * sm_count())
        parts <<= 1;
    const int per = (N + parts - 1) / parts;
    const int chans = SCAN_THREADS / parts;
    const dim3 grid((inner + chans - 1) / chans, R);
    const size_t smem = (SCAN_STAGES * (size_t)SCAN_TILE * (2 * N + 3 * chans) + (size_t)SCAN_TILE * (SCAN_THREADS + chans)) * sizeof(float);
    const int wide = (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dt_raw) | reinterpret_cast<uintptr_t>(bc) |
                        reinterpret_cast<uintptr_t>(z)) & 15) == 0 && ldx % 4 == 0 && lddt % 4 == 0 && ldbc % 4 == 0 &&
                      ldz % 4 == 0 && N % 2 == 0 && chans % 4 == 0 && inner % 4 == 0) ? 1 : 0;
#define DLM_SEL(NPT, TOUT)                                                                                           \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(selective_scan_kernel<NPT, TOUT>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                 (int)smem);                                                                         \
        selective_scan_kernel<NPT, TOUT><<<grid, SCAN_THREADS, smem, stream>>>(                                      \
            x, ldx, dt_raw, lddt, bc, ldbc, z, ldz, dt_bias, A_log, D, state, cu_q, state_slot,                      \
            static_cast<TOUT*>(out), ldo, inner, N, parts, wide);                                                       \
    } while (0)
#define DLM_SEL_T(NPT)                                                                 \
    do {                                                                               \
        if (out_dtype == F32) DLM_SEL(NPT, float); else DLM_SEL(NPT, __nv_bfloat16);   \
    } while (0)
    if (per <= 1) DLM_SEL_T(1);
    else if (per <= 2) DLM_SEL_T(2);
    else if (per <= 4) DLM_SEL_T(4);
    else DLM_SEL_T(8);
#undef DLM_SEL_T
#undef DLM_SEL
    check_launch("selective_scan");
}

void qk_norm_write(const float* qkv, int ld, const int32_t* positions, const float* qn_w, const float* kn_w, float eps,
                   float temp_coef, int temp_every, const int32_t* slots, void* q_out, void* k_cache, void* v_cache,
                   int T, int nh, int nkv, int d, int dv, int D, int page_size, int total_pages, int dtype,
                   cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(D >= d && D >= dv && d >= 1 && dv >= 1, "qk_norm_write: the stored head size must hold keys and values");
    DLM_CHECK(temp_every >= 0, "qk_norm_write: the temperature's period must not be negative");
    int* err = error_flag_ptr();
    if (dtype == F32)
        launch_dep(qk_norm_write_kernel<float>, dim3(T), dim3(256), 0, stream, qkv, ld, positions, qn_w, kn_w, eps,
                   temp_coef, temp_every, slots, static_cast<float*>(q_out), static_cast<float*>(k_cache),
                   static_cast<float*>(v_cache), nh, nkv, d, dv, D, page_size, total_pages, err);
    else
        launch_dep(qk_norm_write_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, qkv, ld, positions, qn_w, kn_w,
                   eps, temp_coef, temp_every, slots, static_cast<__nv_bfloat16*>(q_out),
                   static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), nh, nkv, d, dv, D,
                   page_size, total_pages, err);
    check_launch("qk_norm_write");
}

void rotate_heads(float* x, int ld, const int32_t* positions, const float* inv_freq, int rot_dims, int T, int heads,
                  int dim, int off_a, float scale_a, int off_b, float scale_b, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim, "rotate_heads: rot_dims must be even, at most dim");
    DLM_CHECK(rot_dims == 0 || inv_freq != nullptr, "rotate_heads: a rotation needs its frequencies");
    const int threads = 2 * heads * dim >= 1024 ? 256 : 128;
    launch_dep(rotate_heads_kernel, dim3(T), dim3(threads), sizeof(float) * (rot_dims > 0 ? rot_dims : 1), stream, x, ld,
               positions, inv_freq, rot_dims, heads, dim, off_a, scale_a, off_b, scale_b);
    check_launch("rotate_heads");
}

void branch_norm_add(float* resid, const float* a, const float* wa, const float* b, const float* wb, float eps,
                     float coef, int T, int H, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(a != nullptr && wa != nullptr && (b == nullptr || wb != nullptr), "branch_norm_add: a branch needs its weight");
    launch_dep(branch_norm_add_kernel, dim3(T), dim3(H >= 1024 ? 256 : 128), 0, stream, resid, a, wa, b, wb, eps, coef, H);
    check_launch("branch_norm_add");
}

void rmsnorm_pair(const float* x, const float* wa, const float* wb, void* out_a, void* out_b, int T, int H, float eps,
                  int out_dtype, cudaStream_t stream) {
    if (T <= 0) return;
    const int threads = H >= 1024 ? 256 : 128;
    if (out_dtype == F32)
        launch_dep(rmsnorm_pair_kernel<float>, dim3(T), dim3(threads), 0, stream, x, wa, wb, static_cast<float*>(out_a),
                   static_cast<float*>(out_b), H, eps);
    else
        launch_dep(rmsnorm_pair_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, x, wa, wb,
                   static_cast<__nv_bfloat16*>(out_a), static_cast<__nv_bfloat16*>(out_b), H, eps);
    check_launch("rmsnorm_pair");
}

void concat_rows(const float* a, const float* b, void* out, int T, int H, int out_dtype, cudaStream_t stream) {
    if (T <= 0) return;
    if (out_dtype == F32)
        launch_dep(concat_rows_kernel<float>, dim3(T), dim3(256), 0, stream, a, b, static_cast<float*>(out), H);
    else
        launch_dep(concat_rows_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, a, b,
                   static_cast<__nv_bfloat16*>(out), H);
    check_launch("concat_rows");
}

}  // namespace dlmk
