// Parts of layers that mix several kinds of sublayers, with the small kernels that surround them.
//
//   streams_norm      several copies of the residual stream (hyper-connections): the streams take a sublayer's
//                     output in (X_t ← Σ_s mix[s,t] X_s + out_t y), and the next sublayer's input is the layer norm
//                     (mean and variance, a weight, no bias) of Σ_s in_s X_s; with one stream and no coefficients it
//                     is a plain layer norm
//   streams_expand    the embedding's rows copied into every stream
//   conv_qk_store     a short causal convolution over time on every channel of q, k, v (its last inputs are a
//                     sequence's state), rotation of dim i with dim i + dims/2 over the first dims of every head,
//                     a weightless rms norm of q and k per head, q out, k / v to pages
//   gla               gated linear attention: S_t = diag(α_t) S_{t-1} + k_t v_tᵀ, o_t = S_tᵀ q_t with a decay per key
//                     channel from a low-rank projection, rms norm with a weight per head, gate silu(g)
//   gelu_tanh, clamped_glu     activations of feed-forwards
//   moe_select        sigmoid router: choice among the best groups of experts with a correction, weights without it
//   moe_plan / moe_up / moe_down / moe_combine      the chosen experts' products over token lists sorted by expert
//
// Everything but the experts' products is computed in 32-bit (FFMA, expf / tanhf / sqrtf / division without
// fast-math); stores round to the activation type. States are 32-bit. Every output row is reduced in an order that
// depends on its own sequence only, never on the batch or on how the tokens were cut into steps.
#include "common.cuh"
#include "flash_common.cuh"

SP_API const char* sp_hybrid_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(hybrid)

__device__ __forceinline__ float hy_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float hy_silu(float x) { return x / (1.0f + expf(-x)); }

// ============================================================== streams: update, mix and layer norm
#define HC_MAX_STREAMS 8
struct HcArgs {
    float* x;                 // [T][S·W] the streams of every token, updated in place when ``y`` is given
    float* y;                 // [T][W] a sublayer's output, or null; left zeroed for the next sublayer to add into
    const float* mix;         // [S][S] (from, to), or null: every stream keeps itself
    const float* outc;        // [S] how much of y each stream takes, or null: all of it
    const float* inc;         // [S] coefficients of the norm's input, or null: the sum of the streams
    const void* w; int w_dt;  // the norm's weight [W], or null: no norm, the update only
    void* out; int out_dt;    // [n_rows][W]
    const int* rows;          // optional gather of token rows (without ``y`` only)
    int n_rows, S, W;
    float eps;
};

// One block per token row; a thread takes groups of VEC neighbouring columns (VEC 4: 16-byte loads and stores, for
// widths that are multiples of four), so that a row's loads are all in flight at once. The norm's input waits in
// shared memory between the passes (mean, then the mean of the squared deviations, then the store); each thread reads
// back only what it wrote.
template <int VEC, int SMAX>
__global__ void __launch_bounds__(256, SMAX <= 2 ? 6 : SMAX <= 4 ? 3 : 1) streams_norm_kernel(HcArgs a) {
    extern __shared__ __align__(16) float u[];         // [W rounded up to 4]
    __shared__ float red[32];
    __shared__ float cm[HC_MAX_STREAMS * HC_MAX_STREAMS], co[HC_MAX_STREAMS], ci[HC_MAX_STREAMS];
    const int S = a.S, W = a.W;
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) cm[i] = a.mix ? a.mix[i] : (i / S == i % S ? 1.0f : 0.0f);
    if (threadIdx.x < S) {
        co[threadIdx.x] = a.outc ? a.outc[threadIdx.x] : 1.0f;
        ci[threadIdx.x] = a.inc ? a.inc[threadIdx.x] : 1.0f;
    }
    __syncthreads();
    const int r = blockIdx.x;
    const size_t row = a.rows ? (size_t)a.rows[r] : (size_t)r;
    float* xr = a.x + row * S * W;
    float part = 0.0f;
    for (int c = threadIdx.x * VEC; c < W; c += blockDim.x * VEC) {
        float xs[SMAX][VEC];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) {
            if (s >= S) break;
            if (VEC == 4) {
                const float4 v = *(const float4*)(xr + (size_t)s * W + c);
                xs[s][0] = v.x; xs[s][1] = v.y; xs[s][2] = v.z; xs[s][VEC - 1] = v.w;
            } else {
                xs[s][0] = xr[(size_t)s * W + c];
            }
        }
        if (a.y) {
            float yv[VEC];
            if (VEC == 4) {
                const float4 v = *(const float4*)(a.y + row * W + c);
                yv[0] = v.x; yv[1] = v.y; yv[2] = v.z; yv[VEC - 1] = v.w;
                *(float4*)(a.y + row * W + c) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            } else {
                yv[0] = a.y[row * W + c];
                a.y[row * W + c] = 0.0f;
            }
            float nx[SMAX][VEC];
#pragma unroll
            for (int t = 0; t < SMAX; ++t) {
                if (t >= S) break;
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    float v = 0.0f;
#pragma unroll
                    for (int s = 0; s < SMAX; ++s)
                        if (s < S) v = fmaf(cm[s * S + t], xs[s][i], v);
                    nx[t][i] = fmaf(co[t], yv[i], v);
                }
            }
#pragma unroll
            for (int t = 0; t < SMAX; ++t) {
                if (t >= S) break;
#pragma unroll
                for (int i = 0; i < VEC; ++i) xs[t][i] = nx[t][i];
                if (VEC == 4) *(float4*)(xr + (size_t)t * W + c) = make_float4(nx[t][0], nx[t][1], nx[t][2], nx[t][VEC - 1]);
                else xr[(size_t)t * W + c] = nx[t][0];
            }
        }
        if (a.w) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                float v = 0.0f;
#pragma unroll
                for (int s = 0; s < SMAX; ++s)
                    if (s < S) v = fmaf(ci[s], xs[s][i], v);
                u[c + i] = v;
                part += v;
            }
        }
    }
    if (!a.w) return;
    const float mean = sp_block_sum(part, red) / (float)W;
    float dev = 0.0f;
    for (int c = threadIdx.x * VEC; c < W; c += blockDim.x * VEC)
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const float dlt = u[c + i] - mean;
            dev = fmaf(dlt, dlt, dev);
        }
    const float var = sp_block_sum(dev, red) / (float)W;
    const float inv = 1.0f / sqrtf(var + a.eps);
    for (int c = threadIdx.x * VEC; c < W; c += blockDim.x * VEC) {
        float o[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] = (u[c + i] - mean) * inv * sp_ld_dt(a.w, a.w_dt, c + i);
        if (VEC == 4 && a.out_dt == SP_DT_F32) {
            *(float4*)((float*)a.out + (size_t)r * W + c) = make_float4(o[0], o[1], o[2], o[VEC - 1]);
        } else if (VEC == 4) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[VEC - 1]);
            *(uint2*)((__nv_bfloat16*)a.out + (size_t)r * W + c) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
        } else {
            sp_st_dt(a.out, a.out_dt, (size_t)r * W + c, o[0]);
        }
    }
}

static SpPerDevice streams_norm_ready;

SP_API int sp_streams_norm(float* x, float* y, const float* mix, const float* outc, const float* inc, const void* w,
                           int w_dt, void* out, int out_dt, const int* rows, int n_rows, int S, int W, float eps,
                           cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (S < 1 || S > HC_MAX_STREAMS) SP_FAIL("streams_norm: %d streams, this kernel takes 1 to %d", S, HC_MAX_STREAMS);
    if (y && rows) SP_FAIL("streams_norm: an update runs over all rows");
    const size_t smem = (size_t)((W + 3) / 4 * 4) * sizeof(float);
    if (smem > 200 * 1024) SP_FAIL("streams_norm: a row of %d does not fit shared memory", W);
    if (smem > 48 * 1024 && !streams_norm_ready.done()) {
        if (cudaFuncSetAttribute(streams_norm_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(streams_norm_kernel<4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(streams_norm_kernel<1, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(streams_norm_kernel<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(streams_norm_kernel<1, HC_MAX_STREAMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(streams_norm_kernel<4, HC_MAX_STREAMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            SP_FAIL("streams_norm: cannot raise the shared memory limit");
        streams_norm_ready.mark();
    }
    HcArgs a{x, y, mix, outc, inc, w, w_dt, out, out_dt, rows, n_rows, S, W, eps};
    const bool wide = W % 4 == 0 && ((((uintptr_t)x) | ((uintptr_t)y) | ((uintptr_t)out)) & 15) == 0;
    const int groups = wide ? W / 4 : W;
    int threads = (groups + 31) / 32 * 32;
    threads = threads < 64 ? 64 : threads > 256 ? 256 : threads;
    if (wide && S <= 2) streams_norm_kernel<4, 2><<<n_rows, threads, smem, stream>>>(a);
    else if (S <= 2) streams_norm_kernel<1, 2><<<n_rows, threads, smem, stream>>>(a);
    else if (wide && S <= 4) streams_norm_kernel<4, 4><<<n_rows, threads, smem, stream>>>(a);
    else if (wide) streams_norm_kernel<4, HC_MAX_STREAMS><<<n_rows, threads, smem, stream>>>(a);
    else if (S <= 4) streams_norm_kernel<1, 4><<<n_rows, threads, smem, stream>>>(a);
    else streams_norm_kernel<1, HC_MAX_STREAMS><<<n_rows, threads, smem, stream>>>(a);
    SP_CHECK_LAUNCH("streams_norm");
    return 0;
}

__global__ void streams_expand_kernel(const float* __restrict__ h, float* __restrict__ x, size_t T, int S, int W) {
    const size_t n = T * (size_t)S * W;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / ((size_t)S * W);
        x[e] = h[t * W + e % W];
    }
}

SP_API int sp_streams_expand(const float* h, float* x, int T, int S, int W, cudaStream_t stream) {
    if (T <= 0) return 0;
    const size_t n = (size_t)T * S * W;
    const size_t want = (n + 255) / 256;
    streams_expand_kernel<<<(unsigned)(want > 148 * 16 ? 148 * 16 : want), 256, 0, stream>>>(h, x, (size_t)T, S, W);
    SP_CHECK_LAUNCH("streams_expand");
    return 0;
}

// ============================================================== short convolution, rotation, unit rms, cache write
// qkv row (32-bit) = [q: nh·d | k: nkv·d | v: nkv·vd] = C channels (``v_from_k``: no v channels; the values are the
// keys as they leave the convolution, before their rotation). The convolution of channel c at a token reads the
// channel's projected values of the token and of the taps−1 tokens before it: from this step's rows where the step
// has them, from state[slot][r][c] (r = 0 the oldest) where they came with earlier steps, zeros before the sequence's
// start (a fresh slot's state is zero). One block per token, a warp per head; the head's values pass through shared
// memory so that a lane reaches both halves of a rotated pair.
#define CQ_MAX_DIM 256
#define CQ_WARPS 4
#define CQ_MAX_TAPS 8
struct CqArgs {
    const float* qkv; int ld;
    const void* conv; int conv_dt; int taps;      // [C][taps]; taps 1 and conv null: no convolution
    float* state; int n_slots;                     // [slots][taps−1][C]
    const float* inv_freq; int rd;                 // rd 0: no rotation
    void* q_out; int q_dt;
    void* kpool; void* vpool; int cache_dt;
    const int* token_seq; const int* positions; const int* seq_row; const int* page_table; int max_pages, page_size;
    const int* seq_start; const int* seq_slot;
    int T, nh, nkv, d, vd;
    float eps, v_scale;
    int unit_rms;                                  // 1: q and k leave with unit rms per head
    int save_inline;                               // 1: every sequence brings one token, so the token's block also shifts the state
    int v_from_k;                                  // 1: no v channels: the values are the convolved keys, before their rotation
    SpRange rg;
};

__device__ __forceinline__ float cq_conv(const CqArgs& a, int t, int local, int slot, int c, int C) {
    const float cur = a.qkv[(size_t)t * a.ld + c];
    if (a.taps <= 1) return a.conv ? cur * sp_ld_dt(a.conv, a.conv_dt, c) : cur;
    float u[CQ_MAX_TAPS];
    const int n = a.taps - 1;
    float* st = a.state + (size_t)slot * n * C + c;
#pragma unroll
    for (int j = 0; j < CQ_MAX_TAPS; ++j) {
        if (j >= a.taps) break;
        const int l = local - n + j;               // place of tap j among the step's tokens of this sequence
        u[j] = l >= 0 ? a.qkv[(size_t)(t - n + j) * a.ld + c] : st[(size_t)(n + l) * C];
    }
    float y = 0.0f;
#pragma unroll
    for (int j = 0; j < CQ_MAX_TAPS; ++j) {
        if (j >= a.taps) break;
        y = fmaf(sp_ld_dt(a.conv, a.conv_dt, (size_t)c * a.taps + j), u[j], y);
    }
    if (a.save_inline) {
        // local is 0 here, so u[j] is the state's row j for j < n, and the token's own value last
#pragma unroll
        for (int r = 0; r < CQ_MAX_TAPS - 1; ++r)
            if (r < n) st[(size_t)r * C] = u[r + 1];
    }
    return y;
}

__global__ void __launch_bounds__(CQ_WARPS * 32) conv_qk_store_kernel(CqArgs a) {
    __shared__ float hv[CQ_WARPS][CQ_MAX_DIM];
    __shared__ float cs[2][CQ_MAX_DIM / 2];
    const int t = blockIdx.x;
    if (t >= a.T) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = a.token_seq[t];
    const int pos = a.positions[t];
    const int local = t - a.seq_start[s];
    const int slot = a.seq_slot[s];
    if (a.taps > 1 && (slot < 0 || slot >= a.n_slots)) return;
    const int half = a.rd >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * a.inv_freq[i];
        cs[0][i] = cosf(ang);
        cs[1][i] = sinf(ang);
    }
    __syncthreads();
    const int d = a.d, vd = a.vd, nh = a.nh, nkv = a.nkv;
    const int C = (nh + nkv) * d + (a.v_from_k ? 0 : nkv * vd);
    bool place = true;
    int page = 0;
    {
        const int row = a.seq_row[s];
        if (!sp_index_ok(row, a.rg.n_rows, a.rg, 402) || !sp_index_ok(pos / a.page_size, a.max_pages, a.rg, 403)) place = false;
        else {
            page = a.page_table[(size_t)row * a.max_pages + pos / a.page_size];
            place = sp_index_ok(page, a.rg.n_pages, a.rg, 401);
        }
    }
    const int off = pos % a.page_size;
    for (int hh = warp; hh < nh + (a.v_from_k ? 1 : 2) * nkv; hh += CQ_WARPS) {
        const bool is_v = hh >= nh + nkv;
        const int size = is_v ? vd : d;
        const int cb = is_v ? (nh + nkv) * d + (hh - nh - nkv) * vd : hh * d;
        __syncwarp();
        for (int i = lane; i < size; i += 32) hv[warp][i] = cq_conv(a, t, local, slot, cb + i, C);
        __syncwarp();
        if (is_v) {
            if (place) {
                const size_t vb = (((size_t)page * nkv + (hh - nh - nkv)) * a.page_size + off) * vd;
                for (int i = lane; i < vd; i += 32) sp_st_dt(a.vpool, a.cache_dt, vb + i, hv[warp][i] * a.v_scale);
            }
            continue;
        }
        if (a.v_from_k && hh >= nh && place) {
            const size_t vb = (((size_t)page * nkv + (hh - nh)) * a.page_size + off) * d;
            for (int i = lane; i < d; i += 32) sp_st_dt(a.vpool, a.cache_dt, vb + i, hv[warp][i] * a.v_scale);
            __syncwarp();
        }
        for (int i = lane; i < half; i += 32) {
            const float x0 = hv[warp][i], x1 = hv[warp][i + half];
            hv[warp][i] = x0 * cs[0][i] - x1 * cs[1][i];
            hv[warp][i + half] = x1 * cs[0][i] + x0 * cs[1][i];
        }
        __syncwarp();
        float inv = 1.0f;
        if (a.unit_rms) {
            float ss = 0.0f;
            for (int i = lane; i < d; i += 32) ss = fmaf(hv[warp][i], hv[warp][i], ss);
            ss = sp_warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)d + a.eps);
        }
        if (hh < nh) {
            for (int i = lane; i < d; i += 32) sp_st_dt(a.q_out, a.q_dt, (size_t)t * nh * d + (size_t)hh * d + i, hv[warp][i] * inv);
        } else if (place) {
            const size_t kb = (((size_t)page * nkv + (hh - nh)) * a.page_size + off) * d;
            for (int i = lane; i < d; i += 32) sp_st_dt(a.kpool, a.cache_dt, kb + i, hv[warp][i] * inv);
        }
    }
}

// The same for sizes that are multiples of four (head sizes, half the rotated dims, the row strides): a lane takes four
// neighbouring dims with 16-byte loads and 8- or 16-byte stores, eight warps share a token's heads.
#define CQV_WARPS 8
__device__ __forceinline__ void cq_store4(void* p, int dt, size_t i, float4 v) {
    if (dt == SP_DT_F32) {
        *(float4*)((float*)p + i) = v;
    } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        *(uint2*)((__nv_bfloat16*)p + i) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
    }
}

__global__ void __launch_bounds__(CQV_WARPS * 32) conv_qk_store_vec_kernel(CqArgs a) {
    __shared__ __align__(16) float hv[CQV_WARPS][CQ_MAX_DIM];
    __shared__ __align__(16) float cs[2][CQ_MAX_DIM / 2];
    const int t = blockIdx.x;
    if (t >= a.T) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = a.token_seq[t];
    const int pos = a.positions[t];
    const int local = t - a.seq_start[s];
    const int slot = a.seq_slot[s];
    if (a.taps > 1 && (slot < 0 || slot >= a.n_slots)) return;
    const int half = a.rd >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * a.inv_freq[i];
        cs[0][i] = cosf(ang);
        cs[1][i] = sinf(ang);
    }
    __syncthreads();
    const int d = a.d, vd = a.vd, nh = a.nh, nkv = a.nkv, n = a.taps - 1;
    const int C = (nh + nkv) * d + (a.v_from_k ? 0 : nkv * vd);
    bool place = true;
    int page = 0;
    {
        const int row = a.seq_row[s];
        if (!sp_index_ok(row, a.rg.n_rows, a.rg, 402) || !sp_index_ok(pos / a.page_size, a.max_pages, a.rg, 403)) place = false;
        else {
            page = a.page_table[(size_t)row * a.max_pages + pos / a.page_size];
            place = sp_index_ok(page, a.rg.n_pages, a.rg, 401);
        }
    }
    const int off = pos % a.page_size;
    float* st = a.taps > 1 ? a.state + (size_t)slot * n * C : nullptr;
    // a step of few tokens shares a token's heads out over gridDim.y blocks (a head's channels stay with one warp)
    for (int hh = blockIdx.y * CQV_WARPS + warp; hh < nh + (a.v_from_k ? 1 : 2) * nkv; hh += CQV_WARPS * gridDim.y) {
        const bool is_v = hh >= nh + nkv;
        const int size = is_v ? vd : d;
        const int cb = is_v ? (nh + nkv) * d + (hh - nh - nkv) * vd : hh * d;
        __syncwarp();
        for (int i = lane * 4; i < size; i += 128) {
            const int c = cb + i;
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int j = 0; j < a.taps; ++j) {
                const int l = local - n + j;
                const float4 u = l >= 0 ? *(const float4*)(a.qkv + (size_t)(t - n + j) * a.ld + c) : *(const float4*)(st + (size_t)(n + l) * C + c);
                if (a.conv) {
                    acc.x = fmaf(sp_ld_dt(a.conv, a.conv_dt, (size_t)c * a.taps + j), u.x, acc.x);
                    acc.y = fmaf(sp_ld_dt(a.conv, a.conv_dt, (size_t)(c + 1) * a.taps + j), u.y, acc.y);
                    acc.z = fmaf(sp_ld_dt(a.conv, a.conv_dt, (size_t)(c + 2) * a.taps + j), u.z, acc.z);
                    acc.w = fmaf(sp_ld_dt(a.conv, a.conv_dt, (size_t)(c + 3) * a.taps + j), u.w, acc.w);
                } else {
                    acc = u;
                }
                if (a.save_inline && j >= 1) *(float4*)(st + (size_t)(j - 1) * C + c) = u;     // local is 0: row j was read first
            }
            *(float4*)&hv[warp][i] = acc;
        }
        __syncwarp();
        if (is_v) {
            if (place) {
                const size_t vb = (((size_t)page * nkv + (hh - nh - nkv)) * a.page_size + off) * vd;
                for (int i = lane * 4; i < vd; i += 128) {
                    const float4 v = *(const float4*)&hv[warp][i];
                    cq_store4(a.vpool, a.cache_dt, vb + i, make_float4(v.x * a.v_scale, v.y * a.v_scale, v.z * a.v_scale, v.w * a.v_scale));
                }
            }
            continue;
        }
        if (a.v_from_k && hh >= nh && place) {
            const size_t vb = (((size_t)page * nkv + (hh - nh)) * a.page_size + off) * d;
            for (int i = lane * 4; i < d; i += 128) {
                const float4 v = *(const float4*)&hv[warp][i];
                cq_store4(a.vpool, a.cache_dt, vb + i, make_float4(v.x * a.v_scale, v.y * a.v_scale, v.z * a.v_scale, v.w * a.v_scale));
            }
            __syncwarp();
        }
        for (int i = lane * 4; i < half; i += 128) {
            const float4 x0 = *(const float4*)&hv[warp][i], x1 = *(const float4*)&hv[warp][i + half];
            const float4 co = *(const float4*)&cs[0][i], si = *(const float4*)&cs[1][i];
            *(float4*)&hv[warp][i] = make_float4(x0.x * co.x - x1.x * si.x, x0.y * co.y - x1.y * si.y, x0.z * co.z - x1.z * si.z, x0.w * co.w - x1.w * si.w);
            *(float4*)&hv[warp][i + half] = make_float4(x1.x * co.x + x0.x * si.x, x1.y * co.y + x0.y * si.y, x1.z * co.z + x0.z * si.z, x1.w * co.w + x0.w * si.w);
        }
        __syncwarp();
        float inv = 1.0f;
        if (a.unit_rms) {
            float ss = 0.0f;
            for (int i = lane * 4; i < d; i += 128) {
                const float4 v = *(const float4*)&hv[warp][i];
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
            ss = sp_warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)d + a.eps);
        }
        if (hh >= nh && !place) continue;
        void* dst = hh < nh ? a.q_out : a.kpool;
        const int dt = hh < nh ? a.q_dt : a.cache_dt;
        const size_t base = hh < nh ? (size_t)t * nh * d + (size_t)hh * d : (((size_t)page * nkv + (hh - nh)) * a.page_size + off) * d;
        for (int i = lane * 4; i < d; i += 128) {
            const float4 v = *(const float4*)&hv[warp][i];
            cq_store4(dst, dt, base + i, make_float4(v.x * inv, v.y * inv, v.z * inv, v.w * inv));
        }
    }
}

// the state after a step of several tokens per sequence: the last taps−1 projected values of each sequence, the
// older ones moved down where the step brought fewer (rows ascending: a row only reads rows above itself)
__global__ void conv_state_save_kernel(CqArgs a, int B, int C) {
    const int s = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (s >= B || c >= C) return;
    const int slot = a.seq_slot[s];
    if (slot < 0 || slot >= a.n_slots) return;
    const int t0 = a.seq_start[s], cnt = a.seq_start[s + 1] - t0, n = a.taps - 1;
    float* st = a.state + (size_t)slot * n * C + c;
    for (int r = 0; r < n; ++r) {
        const int l = cnt - n + r;
        st[(size_t)r * C] = l >= 0 ? a.qkv[(size_t)(t0 + l) * a.ld + c] : st[(size_t)(r + cnt) * C];
    }
}

SP_API int sp_conv_qk_store(const float* qkv, int ld, const void* conv, int conv_dt, int taps, float* state, int n_slots,
                            const float* inv_freq, int rd, void* q_out, int q_dt, void* kpool, void* vpool, int cache_dt,
                            const int* token_seq, const int* positions, const int* seq_row, const int* page_table,
                            int max_pages, int page_size, const int* seq_start, const int* seq_slot, int T, int B, int nh,
                            int nkv, int d, int vd, float eps, float v_scale, int unit_rms, int all_single,
                            int v_from_k, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || d > CQ_MAX_DIM || vd <= 0 || vd > CQ_MAX_DIM) SP_FAIL("conv_qk_store: head sizes %d / %d are beyond %d", d, vd, CQ_MAX_DIM);
    if (taps < 1 || taps > CQ_MAX_TAPS) SP_FAIL("conv_qk_store: %d taps, this kernel takes 1 to %d", taps, CQ_MAX_TAPS);
    if (taps > 1 && (!conv || !state)) SP_FAIL("conv_qk_store: a convolution needs its weights and a state");
    if (rd < 0 || (rd & 1) || rd > d) SP_FAIL("conv_qk_store: %d rotated dims do not fit a head of %d", rd, d);
    if (v_from_k && vd != d) SP_FAIL("conv_qk_store: values that are the keys have the keys' size %d, not %d", d, vd);
    CqArgs a{qkv, ld, conv, conv_dt, taps, state, n_slots, inv_freq, rd, q_out, q_dt, kpool, vpool, cache_dt,
             token_seq, positions, seq_row, page_table, max_pages, page_size, seq_start, seq_slot, T, nh, nkv, d, vd,
             eps, v_scale, unit_rms, (all_single && taps > 1) ? 1 : 0, v_from_k ? 1 : 0, sp_range_host};
    const bool wide = d % 4 == 0 && vd % 4 == 0 && (rd / 2) % 4 == 0 && ld % 4 == 0 &&
                      ((((uintptr_t)qkv) | ((uintptr_t)state) | ((uintptr_t)q_out) | ((uintptr_t)kpool) | ((uintptr_t)vpool)) & 15) == 0;
    const int head_rows = nh + (v_from_k ? 1 : 2) * nkv;
    const int by_heads = (head_rows + CQV_WARPS - 1) / CQV_WARPS, by_sms = 296 / (T < 296 ? T : 296);
    const int shares = T >= 148 ? 1 : (by_heads < by_sms ? by_heads : by_sms);
    if (wide) conv_qk_store_vec_kernel<<<dim3(T, shares), CQV_WARPS * 32, 0, stream>>>(a);
    else conv_qk_store_kernel<<<T, CQ_WARPS * 32, 0, stream>>>(a);
    SP_CHECK_LAUNCH("conv_qk_store");
    if (taps > 1 && !all_single) {
        const int C = (nh + nkv) * d + (v_from_k ? 0 : nkv * vd);
        conv_state_save_kernel<<<dim3(B, (C + 127) / 128), 128, 0, stream>>>(a, B, C);
        SP_CHECK_LAUNCH("conv_state_save");
    }
    return 0;
}

// ============================================================== gated linear attention
// proj row (32-bit) = [q: H·d | k: H·d | v: H·vd | g: H·vd | r: rank]. The decay of key channel e of head h at a
// token is α = sigmoid(z)^(1/τ) = exp(logsigmoid(z) / τ) with z = a2[h·d+e, :] · r + b[h·d+e].
struct GlaArgs {
    const float* proj; int ld;
    float* state; int n_slots;           // [slots][H][d][vd]
    const void* a2; const void* a2b; const void* nw; int w_dt;    // [H·d][rank], [H·d], norm weight [vd]
    float* o_raw;                        // [T][H·vd] (the step kernel's raw outputs)
    void* out; int out_dt;               // [T][H·vd]
    const int* seq_start; const int* seq_slot;
    int B, H, d, vd, rank;
    float inv_tau, eps, out_scale;
};

__device__ __forceinline__ float gla_alpha(float z, float inv_tau) {
    const float ls = fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));       // log sigmoid(z)
    return expf(ls * inv_tau);
}

// Token by token. One CTA per (sequence, head): the state S [d][vd] lives in shared memory for the whole step; thread
// (j, y) owns column j of the rows i ≡ y (mod DY); the DY partial sums of a column are added in the order of y.
__global__ void gla_scan_kernel(GlaArgs a, int vdr, int DY) {
    extern __shared__ float sm[];
    const int d = a.d, vd = a.vd, rank = a.rank;
    float* S = sm;                                   // [d][vd]
    float* qs = S + (size_t)d * vd;                  // q/√d [d]
    float* ks = qs + d;                              // k [d]
    float* al = ks + d;                              // α [d]
    float* rr = al + d;                              // r [rank]
    float* red = rr + rank;                          // [DY][vdr]
    float* o = red + (size_t)DY * vdr;               // [vdr]
    float* A2 = o + vdr;                             // [d][rank]
    __shared__ float inv_rms;
    const int s = blockIdx.x, h = blockIdx.y;
    const int slot = a.seq_slot[s];
    if (slot < 0 || slot >= a.n_slots) return;
    const int j = threadIdx.x % vdr, y = threadIdx.x / vdr;
    float* gS = a.state + ((size_t)slot * a.H + h) * d * vd;
    for (int e = threadIdx.x; e < d * vd; e += blockDim.x) S[e] = gS[e];
    for (int e = threadIdx.x; e < d * rank; e += blockDim.x) A2[e] = sp_ld_dt(a.a2, a.w_dt, (size_t)h * d * rank + e);
    const float qscale = 1.0f / sqrtf((float)d);
    const int Hd = a.H * d, Hv = a.H * vd;
    for (int t = a.seq_start[s]; t < a.seq_start[s + 1]; ++t) {
        const float* row = a.proj + (size_t)t * a.ld;
        __syncthreads();
        for (int e = threadIdx.x; e < rank; e += blockDim.x) rr[e] = row[2 * Hd + 2 * Hv + e];
        __syncthreads();
        for (int e = threadIdx.x; e < d; e += blockDim.x) {
            qs[e] = row[h * d + e] * qscale;
            ks[e] = row[Hd + h * d + e];
            float z = sp_ld_dt(a.a2b, a.w_dt, h * d + e);
            for (int r = 0; r < rank; ++r) z = fmaf(A2[e * rank + r], rr[r], z);
            al[e] = gla_alpha(z, a.inv_tau);
        }
        __syncthreads();
        float part = 0.0f;
        if (j < vd) {
            const float v = row[2 * Hd + h * vd + j];
            for (int i = y; i < d; i += DY) {
                const float sv = fmaf(al[i], S[i * vd + j], ks[i] * v);
                S[i * vd + j] = sv;
                part = fmaf(sv, qs[i], part);
            }
        }
        red[y * vdr + j] = part;
        __syncthreads();
        if (y == 0) {
            float sum = 0.0f;
            for (int yy = 0; yy < DY; ++yy) sum += red[yy * vdr + j];
            o[j] = j < vd ? sum : 0.0f;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            float ss = 0.0f;
            for (int c = threadIdx.x; c < vd; c += 32) ss = fmaf(o[c], o[c], ss);
            ss = sp_warp_sum(ss);
            if (threadIdx.x == 0) inv_rms = 1.0f / sqrtf(ss / (float)vd + a.eps);
        }
        __syncthreads();
        if (y == 0 && j < vd)
            sp_st_dt(a.out, a.out_dt, (size_t)t * Hv + h * vd + j,
                     o[j] * inv_rms * sp_ld_dt(a.nw, a.w_dt, j) * hy_silu(row[2 * Hd + Hv + h * vd + j]) * a.out_scale);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < d * vd; e += blockDim.x) gS[e] = S[e];
}

// rms norm with the weight, the gate, the scale, the store; grid (T, H)
__global__ void gla_finish_kernel(GlaArgs a) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, h = blockIdx.y;
    const int vd = a.vd, Hv = a.H * vd;
    const float* o = a.o_raw + (size_t)t * Hv + h * vd;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < vd; c += blockDim.x) ss = fmaf(o[c], o[c], ss);
    ss = sp_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)vd + a.eps);
    const float* g = a.proj + (size_t)t * a.ld + 2 * a.H * a.d + Hv + h * vd;
    for (int c = threadIdx.x; c < vd; c += blockDim.x)
        sp_st_dt(a.out, a.out_dt, (size_t)t * Hv + h * vd + c, o[c] * inv * sp_ld_dt(a.nw, a.w_dt, c) * hy_silu(g[c]) * a.out_scale);
}

// A decode step (one token per sequence): the state is streamed once, straight from and to global memory; grid
// (sequences, heads, blocks of 32 value columns), thread (x, y) takes column x of the rows i ≡ y (mod 8); the eight
// partial sums of a column are added in the order of y.
__global__ void __launch_bounds__(256) gla_step_kernel(GlaArgs a) {
    extern __shared__ float sm[];
    const int d = a.d, vd = a.vd, rank = a.rank;
    float* qs = sm;
    float* ks = qs + d;
    float* al = ks + d;
    float* rr = al + d;                    // [rank]
    float* red = rr + rank;                // [8][32]
    const int s = blockIdx.x, h = blockIdx.y;
    const int slot = a.seq_slot[s];
    if (slot < 0 || slot >= a.n_slots) return;
    const int t = a.seq_start[s];
    const int Hd = a.H * d, Hv = a.H * vd;
    const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
    const int j = blockIdx.z * 32 + x;
    const float* row = a.proj + (size_t)t * a.ld;
    const float qscale = 1.0f / sqrtf((float)d);
    for (int e = threadIdx.x; e < rank; e += blockDim.x) rr[e] = row[2 * Hd + 2 * Hv + e];
    __syncthreads();
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        qs[e] = row[h * d + e] * qscale;
        ks[e] = row[Hd + h * d + e];
        float z = sp_ld_dt(a.a2b, a.w_dt, h * d + e);
        for (int r = 0; r < rank; ++r) z = fmaf(sp_ld_dt(a.a2, a.w_dt, ((size_t)h * d + e) * rank + r), rr[r], z);
        al[e] = gla_alpha(z, a.inv_tau);
    }
    __syncthreads();
    float part = 0.0f;
    if (j < vd) {
        const float v = row[2 * Hd + h * vd + j];
        float* gS = a.state + ((size_t)slot * a.H + h) * d * vd + j;
        for (int i0 = y; i0 < d; i0 += 32) {
            float st[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) st[u] = i0 + 8 * u < d ? gS[(size_t)(i0 + 8 * u) * vd] : 0.0f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + 8 * u;
                if (i >= d) break;
                const float sv = fmaf(al[i], st[u], ks[i] * v);
                gS[(size_t)i * vd] = sv;
                part = fmaf(sv, qs[i], part);
            }
        }
    }
    red[y * 32 + x] = part;
    __syncthreads();
    if (y == 0 && j < vd) {
        float sum = 0.0f;
#pragma unroll
        for (int yy = 0; yy < 8; ++yy) sum += red[yy * 32 + x];
        a.o_raw[(size_t)t * Hv + h * vd + j] = sum;
    }
}

// ---- prompts: chunks of GLC tokens, all chunks in parallel. Within a chunk, with B_i = Σ_{u ≤ i} log α_u per key
// channel (counted from the chunk's first token):
//     o_i   = (q_i ⊙ e^{B_i}) · S₀  +  Σ_{j ≤ i} P_ij v_j,      P_ij = Σ_e q_ie k_je e^{B_ie − B_je}
//     S_end = diag(e^{B_last}) S₀  +  Σ_j (k_j ⊙ e^{B_last − B_j}) v_jᵀ
// Every exponent is ≤ 0, so nothing overflows whatever the decays are. Five launches: (1) per (chunk, head) the decays'
// running sums, q ⊙ e^{B}, k ⊙ e^{B_last − B}, e^{B_last} and P; (2) every chunk's own Σ_j (…) v_jᵀ; (3) per (sequence,
// head) the chunks' start states one after the other, element by element, the last one becomes the slot's state;
// (4) every chunk's outputs from its start state; (5) the norm, the gate, the store. A chunk's arithmetic depends on
// where the chunk starts in its step only. Products are tiles out[m][n] = Σ_k a[k][m]·b[k][n] from shared memory,
// k-major, 16 x 16 threads owning 4·MA x 4 outputs each.
#define GLC 64
#define GLC_TS 68              // row stride of arrays that are 64 tokens wide

struct GlcArgs {
    GlaArgs g;
    float* qe; float* ke;      // [T][H·d]
    float* dl;                 // [chunks][H][d]  e^{B_last}
    float* pt;                 // [chunks][H][64][64]  P transposed: pt[j][i]
    float* cs;                 // [chunks][H][d][vd]: (2) the chunk's own sum, (3) turns it into its start state
    int n_chunks;
};

__device__ __forceinline__ bool glc_chunk_of(const GlaArgs& a, int x, int& s, int& t0, int& n) {
    for (s = 0; s < a.B; ++s) {
        const int first = a.seq_start[s], cnt = a.seq_start[s + 1] - first;
        const int nc = (cnt + GLC - 1) / GLC;
        if (x < nc) {
            t0 = first + x * GLC;
            n = min(GLC, cnt - x * GLC);
            return true;
        }
        x -= nc;
    }
    return false;
}

template <int MA>
__device__ __forceinline__ void glc_mm(const float* __restrict__ a, int lda, const float* __restrict__ b, int ldb, int K,
                                       float (&acc)[4 * MA][4], int ty, int tx) {
    for (int k = 0; k < K; ++k) {
        const float4 bv = *(const float4*)(b + (size_t)k * ldb + 4 * tx);
        const float bn[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int i = 0; i < MA; ++i) {
            const float4 av = *(const float4*)(a + (size_t)k * lda + 4 * ty + 64 * i);
            const float am[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int v = 0; v < 4; ++v) acc[4 * i + u][v] = fmaf(am[u], bn[v], acc[4 * i + u][v]);
        }
    }
}

// (1) grid (chunks, H)
__global__ void __launch_bounds__(256) gla_chunk_prep_kernel(GlcArgs c) {
    extern __shared__ __align__(16) float sm[];
    const GlaArgs& a = c.g;
    const int d = a.d, rank = a.rank;
    float* qT = sm;                           // [d][GLC_TS]  q/√d
    float* kT = qT + (size_t)d * GLC_TS;      // [d][GLC_TS]
    float* bT = kT + (size_t)d * GLC_TS;      // [d][GLC_TS]  B
    float* rr = bT + (size_t)d * GLC_TS;      // [GLC][rank]
    int s, t0, n;
    if (!glc_chunk_of(a, blockIdx.x, s, t0, n)) return;
    const int h = blockIdx.y;
    const int Hd = a.H * d, Hv = a.H * a.vd;
    const float qscale = 1.0f / sqrtf((float)d);
    for (int e = threadIdx.x; e < n * rank; e += blockDim.x) rr[e] = a.proj[(size_t)(t0 + e / rank) * a.ld + 2 * Hd + 2 * Hv + e % rank];
    for (int x = threadIdx.x; x < GLC * d; x += blockDim.x) {
        const int i = x / d, e = x % d;
        const bool in = i < n;
        const float* row = a.proj + (size_t)(t0 + (in ? i : 0)) * a.ld;
        qT[e * GLC_TS + i] = in ? row[h * d + e] * qscale : 0.0f;
        kT[e * GLC_TS + i] = in ? row[Hd + h * d + e] : 0.0f;
    }
    __syncthreads();
    // every token's and channel's log decay by all threads, then the running sums by one thread per channel
    for (int x = threadIdx.x; x < GLC * d; x += blockDim.x) {
        const int e = x / GLC, i = x % GLC;
        float la = 0.0f;
        if (i < n) {
            float z = sp_ld_dt(a.a2b, a.w_dt, h * d + e);
            // a warp's threads share the channel: its row of the decay projection comes as one broadcast load each
            for (int r = 0; r < rank; ++r) z = fmaf(sp_ld_dt(a.a2, a.w_dt, ((size_t)h * d + e) * rank + r), rr[i * rank + r], z);
            la = (fminf(z, 0.0f) - log1pf(expf(-fabsf(z)))) * a.inv_tau;
        }
        bT[e * GLC_TS + i] = la;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        float run = 0.0f;
        for (int i = 0; i < GLC; ++i) {
            run += bT[e * GLC_TS + i];
            bT[e * GLC_TS + i] = run;                            // beyond the chunk's tokens: B_last
        }
    }
    __syncthreads();
    // How far the chunk's decays go: where e^{−B} stays far inside the 32-bit range (the usual case), P is the plain
    // product of q ⊙ e^{B} and k ⊙ e^{−B} (two exponentials per token and channel); else every pair takes its own
    // e^{B_i − B_j} ≤ 1, which cannot overflow whatever the decays are.
    __shared__ float red[32];
    float far = 0.0f;
    for (int e = threadIdx.x; e < d; e += blockDim.x) far = fmaxf(far, -bT[e * GLC_TS + GLC - 1]);
    far = sp_block_max(far, red);
    const bool plain = far <= 60.0f;
    // P: thread (ty, tx) owns pairs i = 4ty … 4ty+3, j = 4tx … 4tx+3; blocks above the diagonal stay zero
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float p[4][4] = {};
    if (plain) {
        __syncthreads();
        for (int x = threadIdx.x; x < GLC * d; x += blockDim.x) {
            const int e = x / GLC, i = x % GLC;
            const float b = bT[e * GLC_TS + i];
            qT[e * GLC_TS + i] *= expf(b);
            kT[e * GLC_TS + i] *= expf(-b);
        }
        __syncthreads();
        if (tx <= ty) {
            glc_mm<1>(qT, GLC_TS, kT, GLC_TS, d, p, ty, tx);
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    if (4 * tx + v > 4 * ty + u) p[u][v] = 0.0f;
        }
    } else if (tx <= ty) {
        for (int e = 0; e < d; ++e) {
            const float4 q4 = *(const float4*)(qT + e * GLC_TS + 4 * ty), bi4 = *(const float4*)(bT + e * GLC_TS + 4 * ty);
            const float4 k4 = *(const float4*)(kT + e * GLC_TS + 4 * tx), bj4 = *(const float4*)(bT + e * GLC_TS + 4 * tx);
            const float qi[4] = {q4.x, q4.y, q4.z, q4.w}, bi[4] = {bi4.x, bi4.y, bi4.z, bi4.w};
            const float kj[4] = {k4.x, k4.y, k4.z, k4.w}, bj[4] = {bj4.x, bj4.y, bj4.z, bj4.w};
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    if (4 * tx + v <= 4 * ty + u) p[u][v] = fmaf(qi[u] * kj[v], expf(bi[u] - bj[v]), p[u][v]);
        }
    }
    float* pt = c.pt + ((size_t)blockIdx.x * a.H + h) * GLC * GLC;
#pragma unroll
    for (int v = 0; v < 4; ++v)
        *(float4*)(pt + (size_t)(4 * tx + v) * GLC + 4 * ty) = make_float4(p[0][v], p[1][v], p[2][v], p[3][v]);
    // q ⊙ e^{B}, k ⊙ e^{B_last − B}, e^{B_last}
    for (int x = threadIdx.x; x < n * d; x += blockDim.x) {
        const int i = x / d, e = x % d;
        const float b = bT[e * GLC_TS + i], bl = bT[e * GLC_TS + GLC - 1];
        const float qv = qT[e * GLC_TS + i], kv = kT[e * GLC_TS + i];
        c.qe[(size_t)(t0 + i) * Hd + h * d + e] = plain ? qv : qv * expf(b);
        c.ke[(size_t)(t0 + i) * Hd + h * d + e] = plain ? kv * expf(bl) : kv * expf(bl - b);
    }
    for (int e = threadIdx.x; e < d; e += blockDim.x) c.dl[((size_t)blockIdx.x * a.H + h) * d + e] = expf(bT[e * GLC_TS + GLC - 1]);
}

// (2) grid (chunks, H, column blocks of 64); MA = ceil(d / 64)
template <int MA>
__global__ void __launch_bounds__(256) gla_chunk_sum_kernel(GlcArgs c) {
    extern __shared__ __align__(16) float sm[];
    const GlaArgs& a = c.g;
    const int DP = 64 * MA, d = a.d, vd = a.vd;
    float* kd = sm;                    // [64][DP]
    float* vv = kd + GLC * DP;         // [64][64]
    int s, t0, n;
    if (!glc_chunk_of(a, blockIdx.x, s, t0, n)) return;
    const int h = blockIdx.y, c0 = blockIdx.z * 64;
    const int Hd = a.H * d;
    for (int x = threadIdx.x; x < GLC * DP; x += blockDim.x) {
        const int j = x / DP, e = x % DP;
        kd[x] = (j < n && e < d) ? c.ke[(size_t)(t0 + j) * Hd + h * d + e] : 0.0f;
    }
    for (int x = threadIdx.x; x < GLC * 64; x += blockDim.x) {
        const int j = x / 64, col = c0 + x % 64;
        vv[x] = (j < n && col < vd) ? a.proj[(size_t)(t0 + j) * a.ld + 2 * Hd + h * vd + col] : 0.0f;
    }
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4 * MA][4] = {};
    glc_mm<MA>(kd, DP, vv, 64, GLC, acc, ty, tx);
    float* out = c.cs + ((size_t)blockIdx.x * a.H + h) * d * vd;
#pragma unroll
    for (int i = 0; i < MA; ++i)
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = 4 * ty + 64 * i + u;
            if (e >= d) continue;
#pragma unroll
            for (int v = 0; v < 4; ++v)
                if (c0 + 4 * tx + v < vd) out[(size_t)e * vd + c0 + 4 * tx + v] = acc[4 * i + u][v];
        }
}

// (3) grid (sequences, H, blocks of 256 state elements)
__global__ void __launch_bounds__(256) gla_chunk_scan_kernel(GlcArgs c) {
    const GlaArgs& a = c.g;
    const int s = blockIdx.x, h = blockIdx.y;
    const int x = blockIdx.z * 256 + threadIdx.x;
    if (x >= a.d * a.vd) return;
    const int slot = a.seq_slot[s];
    if (slot < 0 || slot >= a.n_slots) return;
    int first_chunk = 0;
    for (int b = 0; b < s; ++b) first_chunk += (a.seq_start[b + 1] - a.seq_start[b] + GLC - 1) / GLC;
    const int nc = (a.seq_start[s + 1] - a.seq_start[s] + GLC - 1) / GLC;
    float* st = a.state + ((size_t)slot * a.H + h) * a.d * a.vd + x;
    float S = *st;
    const int e = x / a.vd;
    // eight chunks' sums and decays are asked for together (they do not depend on S), then taken in order
    for (int k0 = 0; k0 < nc; k0 += 8) {
        float own[8], dv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (k0 + u < nc) {
                own[u] = c.cs[((size_t)(first_chunk + k0 + u) * a.H + h) * a.d * a.vd + x];
                dv[u] = c.dl[((size_t)(first_chunk + k0 + u) * a.H + h) * a.d + e];
            }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (k0 + u < nc) {
                c.cs[((size_t)(first_chunk + k0 + u) * a.H + h) * a.d * a.vd + x] = S;
                S = fmaf(dv[u], S, own[u]);
            }
    }
    *st = S;
}

// (4) grid (chunks, H, column blocks of 64)
template <int MA>
__global__ void __launch_bounds__(256) gla_chunk_out_kernel(GlcArgs c) {
    extern __shared__ __align__(16) float sm[];
    const GlaArgs& a = c.g;
    const int DP = 64 * MA, d = a.d, vd = a.vd;
    float* qT = sm;                          // [DP][GLC_TS]
    float* S = qT + (size_t)DP * GLC_TS;     // [DP][64]
    float* pT = S + (size_t)DP * 64;         // [64][64]
    float* vv = pT + GLC * 64;               // [64][64]
    int s, t0, n;
    if (!glc_chunk_of(a, blockIdx.x, s, t0, n)) return;
    const int h = blockIdx.y, c0 = blockIdx.z * 64;
    const int Hd = a.H * d, Hv = a.H * vd;
    for (int x = threadIdx.x; x < GLC * DP; x += blockDim.x) {
        const int i = x / DP, e = x % DP;
        qT[e * GLC_TS + i] = (i < n && e < d) ? c.qe[(size_t)(t0 + i) * Hd + h * d + e] : 0.0f;
    }
    const float* cs = c.cs + ((size_t)blockIdx.x * a.H + h) * d * vd;
    for (int x = threadIdx.x; x < DP * 64; x += blockDim.x) {
        const int e = x / 64, col = c0 + x % 64;
        S[x] = (e < d && col < vd) ? cs[(size_t)e * vd + col] : 0.0f;
    }
    const float* pt = c.pt + ((size_t)blockIdx.x * a.H + h) * GLC * GLC;
    for (int x = threadIdx.x; x < GLC * 64; x += blockDim.x) {
        const int j = x / 64, col = c0 + x % 64;
        pT[x] = pt[x];
        vv[x] = (j < n && col < vd) ? a.proj[(size_t)(t0 + j) * a.ld + 2 * Hd + h * vd + col] : 0.0f;
    }
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4][4] = {};
    glc_mm<1>(qT, GLC_TS, S, 64, d, acc, ty, tx);
    glc_mm<1>(pT, 64, vv, 64, GLC, acc, ty, tx);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = 4 * ty + u;
        if (i >= n) continue;
#pragma unroll
        for (int v = 0; v < 4; ++v)
            if (c0 + 4 * tx + v < vd) a.o_raw[(size_t)(t0 + i) * Hv + h * vd + c0 + 4 * tx + v] = acc[u][v];
    }
}

// every region of the scratch starts on 16 bytes (the tiles are stored four floats at a time)
static inline long long glc_up4(long long n) { return (n + 3) / 4 * 4; }

SP_API int sp_gla_chunk_tokens() { return GLC; }
SP_API int sp_gla_chunked_supported(int d, int vd, int rank) { return d > 0 && d <= 128 && vd > 0 && rank > 0 && rank <= 64; }
// floats of scratch the chunked form needs (the raw outputs included)
SP_API long long sp_gla_chunked_scratch_floats(int n_chunks, int T, int H, int d, int vd) {
    return 2LL * glc_up4((long long)T * H * d) + glc_up4((long long)n_chunks * H * d) + (long long)n_chunks * H * GLC * GLC +
           glc_up4((long long)n_chunks * H * d * vd) + (long long)T * H * vd;
}

static SpPerDevice gla_chunk_ready;

SP_API int sp_gla_chunked(const float* proj, int ld, float* state, int n_slots, const void* a2, const void* a2b,
                          const void* nw, int w_dt, float* scratch, void* out, int out_dt, const int* seq_start,
                          const int* seq_slot, int B, int T, int n_chunks, int H, int d, int vd, int rank, float tau,
                          float eps, float out_scale, cudaStream_t stream) {
    if (B <= 0 || T <= 0) return 0;
    if (!sp_gla_chunked_supported(d, vd, rank)) SP_FAIL("gla (chunks): sizes d %d, vd %d, rank %d are outside this kernel's range", d, vd, rank);
    if (!(tau > 0.0f)) SP_FAIL("gla: tau must be positive");
    GlcArgs c;
    c.g = GlaArgs{proj, ld, state, n_slots, a2, a2b, nw, w_dt, nullptr, out, out_dt, seq_start, seq_slot, B, H, d, vd, rank,
                  1.0f / tau, eps, out_scale};
    c.qe = scratch;
    if (((uintptr_t)scratch) & 15) SP_FAIL("gla (chunks): the scratch must start on 16 bytes");
    c.ke = c.qe + glc_up4((long long)T * H * d);
    c.dl = c.ke + glc_up4((long long)T * H * d);
    c.pt = c.dl + glc_up4((long long)n_chunks * H * d);
    c.cs = c.pt + (size_t)n_chunks * H * GLC * GLC;
    c.g.o_raw = c.cs + glc_up4((long long)n_chunks * H * d * vd);
    c.n_chunks = n_chunks;
    const int MA = d <= 64 ? 1 : 2, DP = 64 * MA;
    const size_t smem1 = (3 * (size_t)d * GLC_TS + (size_t)GLC * rank) * sizeof(float);       // two CTAs per SM at d = 128
    const size_t smem2 = ((size_t)GLC * DP + GLC * 64) * sizeof(float);
    const size_t smem4 = ((size_t)DP * GLC_TS + (size_t)DP * 64 + 2 * GLC * 64) * sizeof(float);
    if (!gla_chunk_ready.done()) {
        if (cudaFuncSetAttribute(gla_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(gla_chunk_sum_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(gla_chunk_sum_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(gla_chunk_out_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(gla_chunk_out_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            SP_FAIL("gla (chunks): cannot raise the shared memory limit");
        gla_chunk_ready.mark();
    }
    const int vb = (vd + 63) / 64;
    gla_chunk_prep_kernel<<<dim3(n_chunks, H), 256, smem1, stream>>>(c);
    SP_CHECK_LAUNCH("gla_chunk_prep");
    if (MA == 1) gla_chunk_sum_kernel<1><<<dim3(n_chunks, H, vb), 256, smem2, stream>>>(c);
    else gla_chunk_sum_kernel<2><<<dim3(n_chunks, H, vb), 256, smem2, stream>>>(c);
    SP_CHECK_LAUNCH("gla_chunk_sum");
    gla_chunk_scan_kernel<<<dim3(B, H, (d * vd + 255) / 256), 256, 0, stream>>>(c);
    SP_CHECK_LAUNCH("gla_chunk_scan");
    if (MA == 1) gla_chunk_out_kernel<1><<<dim3(n_chunks, H, vb), 256, smem4, stream>>>(c);
    else gla_chunk_out_kernel<2><<<dim3(n_chunks, H, vb), 256, smem4, stream>>>(c);
    SP_CHECK_LAUNCH("gla_chunk_out");
    gla_finish_kernel<<<dim3(T, H), 128, 0, stream>>>(c.g);
    SP_CHECK_LAUNCH("gla_finish");
    return 0;
}

static SpPerDevice gla_ready;

// mode 0: token by token (any portion); 1: a decode step (needs o_raw)
SP_API int sp_gla(const float* proj, int ld, float* state, int n_slots, const void* a2, const void* a2b, const void* nw,
                  int w_dt, float* o_raw, void* out, int out_dt, const int* seq_start, const int* seq_slot, int B, int H,
                  int d, int vd, int rank, float tau, float eps, float out_scale, int mode, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (d <= 0 || vd <= 0 || vd > 1024 || rank <= 0 || rank > 1024) SP_FAIL("gla: sizes d %d, vd %d, rank %d are outside this kernel's range", d, vd, rank);
    if (!(tau > 0.0f)) SP_FAIL("gla: tau must be positive");
    GlaArgs a{proj, ld, state, n_slots, a2, a2b, nw, w_dt, o_raw, out, out_dt, seq_start, seq_slot, B, H, d, vd, rank,
              1.0f / tau, eps, out_scale};
    if (!gla_ready.done()) {
        if (cudaFuncSetAttribute(gla_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess)
            SP_FAIL("gla: cannot raise the shared memory limit");
        gla_ready.mark();
    }
    if (mode == 1) {
        if (!o_raw) SP_FAIL("gla: a decode step needs room for its raw outputs");
        const size_t smem = ((size_t)3 * d + rank + 256) * sizeof(float);
        if (smem > 48 * 1024) SP_FAIL("gla (step): key size %d is beyond this kernel's range", d);
        gla_step_kernel<<<dim3(B, H, (vd + 31) / 32), 256, smem, stream>>>(a);
        SP_CHECK_LAUNCH("gla_step");
        gla_finish_kernel<<<dim3(B, H), 128, 0, stream>>>(a);
        SP_CHECK_LAUNCH("gla_finish");
        return 0;
    }
    const int vdr = (vd + 31) / 32 * 32;
    int DY = 256 / vdr;
    if (DY < 1) DY = 1;
    if (DY > d) DY = d;
    const size_t smem = ((size_t)d * vd + 3 * d + rank + (size_t)DY * vdr + vdr + (size_t)d * rank) * sizeof(float);
    if (smem > 220 * 1024) SP_FAIL("gla: a state of %d x %d does not fit shared memory", d, vd);
    gla_scan_kernel<<<dim3(B, H), vdr * DY, smem, stream>>>(a, vdr, DY);
    SP_CHECK_LAUNCH("gla");
    return 0;
}

// ============================================================== activations of feed-forwards
__global__ void gelu_tanh_kernel(const void* __restrict__ z, int z_dt, void* __restrict__ out, int out_dt, size_t n) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const float v = sp_ld_dt(z, z_dt, e);
        sp_st_dt(out, out_dt, e, 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v))));
    }
}

SP_API int sp_gelu_tanh(const void* z, int z_dt, void* out, int out_dt, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long want = (n + 255) / 256;
    gelu_tanh_kernel<<<(unsigned)(want > 148 * 16 ? 148 * 16 : want), 256, 0, stream>>>(z, z_dt, out, out_dt, (size_t)n);
    SP_CHECK_LAUNCH("gelu_tanh");
    return 0;
}

// g = min(gate, limit), u = clamp(up, ±limit), out = g · sigmoid(slope · g) · (u + 1); slope 0 asks for silu(gate) · up
__device__ __forceinline__ float hy_clamped_glu(float g, float u, float limit, float slope) {
    if (slope == 0.0f) return g * hy_sigmoid(g) * u;      // the plain gated unit silu(g) · u: no clamp, no shift
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * hy_sigmoid(slope * g) * (u + 1.0f);
}

// gu row = [gate (F) | up (F)]
__global__ void clamped_glu_kernel(const void* __restrict__ gu, int gu_dt, void* __restrict__ out, int out_dt, size_t rows,
                                   int F, float limit, float slope) {
    const size_t n = rows * (size_t)F;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / F;
        const int c = (int)(e % F);
        sp_st_dt(out, out_dt, e, hy_clamped_glu(sp_ld_dt(gu, gu_dt, r * 2 * F + c), sp_ld_dt(gu, gu_dt, r * 2 * F + F + c), limit, slope));
    }
}

SP_API int sp_clamped_glu(const void* gu, int gu_dt, void* out, int out_dt, int rows, int F, float limit, float slope,
                          cudaStream_t stream) {
    if (rows <= 0 || F <= 0) return 0;
    const size_t n = (size_t)rows * F;
    const size_t want = (n + 255) / 256;
    clamped_glu_kernel<<<(unsigned)(want > 148 * 16 ? 148 * 16 : want), 256, 0, stream>>>(gu, gu_dt, out, out_dt, (size_t)rows, F, limit, slope);
    SP_CHECK_LAUNCH("clamped_glu");
    return 0;
}

// ============================================================== the router's choice
// z [T][ldz] (32-bit logits, the first E of a row the experts'). s = sigmoid(z), or with ``softmax`` the softmax of
// the row's E logits; choice c = s + correction (none: s). The weights leave times ``weight_scale``. The experts form ``n_groups`` equal groups of
// neighbours; a group's score is the sum of its two largest c; only experts of the ``keep`` best groups can be chosen
// (n_groups ≤ 1: all). The ``top`` largest allowed c are chosen (among equals the lowest index); their weights are
// their s divided by the sum of those s (+ 1e-20). One warp per token; lane l holds experts l, l+32, ...
#define MS_MAX_E 512
#define MS_WARPS 4
__device__ __forceinline__ void ms_take(float& bv, int& bi, float ov, int oi) {
    if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
}

__global__ void __launch_bounds__(MS_WARPS * 32)
moe_select_kernel(const float* __restrict__ z, const void* __restrict__ corr, int corr_dt, int* __restrict__ ids,
                  float* __restrict__ wts, int T, int E, int ldz, int top, int n_groups, int keep, int softmax,
                  float weight_scale, float* __restrict__ extra) {
    __shared__ float ch[MS_WARPS][MS_MAX_E];        // choice scores; −inf once chosen or not allowed
    __shared__ float sc[MS_WARPS][MS_MAX_E];
    __shared__ float gs[MS_WARPS][MS_MAX_E];        // group scores
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * MS_WARPS + warp;
    if (t >= T) return;
    float zmax = -INFINITY, zsum = 1.0f;
    if (softmax) {
        // scores: the softmax of the logits over all experts (sums in lane order, then across lanes)
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[(size_t)t * ldz + e]);
        zmax = sp_warp_max(zmax);
        float part = 0.0f;
        for (int e = lane; e < E; e += 32) part += expf(z[(size_t)t * ldz + e] - zmax);
        zsum = sp_warp_sum(part);
    }
    for (int e = lane; e < E; e += 32) {
        const float s = softmax ? expf(z[(size_t)t * ldz + e] - zmax) / zsum : hy_sigmoid(z[(size_t)t * ldz + e]);
        sc[warp][e] = s;
        ch[warp][e] = s + (corr ? sp_ld_dt(corr, corr_dt, e) : 0.0f);
    }
    // columns beyond the experts' (ldz > E) pass through: a gate's logit that shared the router's product
    if (extra) for (int e = E + lane; e < ldz; e += 32) extra[(size_t)t * (ldz - E) + (e - E)] = z[(size_t)t * ldz + e];
    __syncwarp();
    if (n_groups > 1) {
        const int gsz = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float b1 = -INFINITY, b2 = -INFINITY;
            for (int e = g * gsz; e < (g + 1) * gsz; ++e) {
                const float c = ch[warp][e];
                if (c > b1) { b2 = b1; b1 = c; }
                else if (c > b2) b2 = c;
            }
            gs[warp][g] = gsz > 1 ? b1 + b2 : b1;
        }
        __syncwarp();
        // the ``keep`` best groups stay; the others' experts leave the choice
        for (int r = 0; r < n_groups - keep; ++r) {
            // drop the worst group still in (among equals the highest index, so that the lowest index wins a place)
            float wv = 0.0f;
            int wi = -1;
            for (int g = lane; g < n_groups; g += 32) {
                const float v = gs[warp][g];
                if (v == INFINITY) continue;                        // already dropped
                if (wi < 0 || v < wv || (v == wv && g > wi)) { wv = v; wi = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, wv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
                if (oi >= 0 && (wi < 0 || ov < wv || (ov == wv && oi > wi))) { wv = ov; wi = oi; }
            }
            if (wi < 0) break;
            for (int e = wi * gsz + lane; e < (wi + 1) * gsz; e += 32) ch[warp][e] = -INFINITY;
            if (lane == 0) gs[warp][wi] = INFINITY;
            __syncwarp();
        }
    }
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) {
        float bv = 0.0f;
        int bi = -1;
        for (int e = lane; e < E; e += 32) {
            const float c = ch[warp][e];
            if (c != -INFINITY) ms_take(bv, bi, c, e);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ms_take(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (bi < 0) bi = 0;                                         // fewer allowed experts than ``top``: refused on the host
        const float s = sc[warp][bi];
        sum += s;
        if (lane == 0) {
            ids[(size_t)t * top + k] = bi;
            wts[(size_t)t * top + k] = s;
            ch[warp][bi] = -INFINITY;
        }
        __syncwarp();
    }
    __syncwarp();
    const float den = sum + 1e-20f;
    for (int k = lane; k < top; k += 32) wts[(size_t)t * top + k] = wts[(size_t)t * top + k] / den * weight_scale;
}

SP_API int sp_moe_select(const float* z, const void* corr, int corr_dt, int* ids, float* wts, int T, int E, int ldz,
                         int top, int n_groups, int keep, int softmax, float weight_scale, float* extra,
                         cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || E > MS_MAX_E) SP_FAIL("moe_select: %d experts, this kernel takes up to %d", E, MS_MAX_E);
    if (ldz < E) SP_FAIL("moe_select: rows of %d logits cannot hold %d experts", ldz, E);
    if (n_groups < 1) n_groups = 1;
    if (E % n_groups) SP_FAIL("moe_select: %d experts do not form %d equal groups", E, n_groups);
    if (n_groups > 1 && (keep < 1 || keep > n_groups)) SP_FAIL("moe_select: %d of %d groups cannot be kept", keep, n_groups);
    const int allowed = n_groups > 1 ? keep * (E / n_groups) : E;
    if (top < 1 || top > allowed) SP_FAIL("moe_select: %d experts cannot be chosen among %d allowed", top, allowed);
    moe_select_kernel<<<(T + MS_WARPS - 1) / MS_WARPS, MS_WARPS * 32, 0, stream>>>(z, corr, corr_dt, ids, wts, T, E, ldz, top, n_groups, keep, softmax, weight_scale, extra);
    SP_CHECK_LAUNCH("moe_select");
    return 0;
}

// ============================================================== the chosen experts' products
// A pair p = token · top + k names one chosen expert of one token. ``moe_plan`` sorts the pairs by expert (pairs of
// one expert in ascending order) and cuts every expert's list into tiles of ME_TM rows: (expert, first place in the
// sorted list, rows); unused entries of the tile table (it is sized for the worst case) say expert −1.
#define ME_TM 32
__global__ void moe_count_kernel(const int* __restrict__ ids, int n_pairs, int* __restrict__ counts) {
    __shared__ int red[32];
    const int e = blockIdx.x;
    int c = 0;
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) c += ids[p] == e;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int sum = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) sum += red[w];
        counts[e] = sum;
    }
}

__global__ void __launch_bounds__(1024)
moe_place_kernel(const int* __restrict__ ids, int n_pairs, const int* __restrict__ counts, int E, int* __restrict__ sorted,
                 int* __restrict__ tiles /* [max_tiles][3] */, int max_tiles, int tm, int padded, int* __restrict__ pos,
                 int* __restrict__ tab_up, int* __restrict__ tab_down, int up_rows, int down_rows) {
    // ``padded``: every expert's rows begin at a tile's first row (the sorted list then has holes, which say -1, and
    // ``pos`` gives every pair its row); ``tab_up`` / ``tab_down``: per tile the row at which the expert's matrices begin
    // in the stacked weights (-1: the tile is not in use), for products that take whole tiles of one expert.
    __shared__ int start, tile0, mine, wsum[32], running;     // blocks of up to 1,024 threads: a pass of the list per 1,024 pairs
    const int e = blockIdx.x;
    if (threadIdx.x == 0) {
        int s = 0, t0 = 0;
        for (int x = 0; x < e; ++x) { s += counts[x]; t0 += (counts[x] + tm - 1) / tm; }
        start = s; tile0 = t0; mine = counts[e]; running = 0;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (int)(blockDim.x >> 5);
    for (int base = 0; base < n_pairs; base += (int)blockDim.x) {
        const int p = base + threadIdx.x;
        const bool hit = p < n_pairs && ids[p] == e;
        const unsigned b = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) wsum[warp] = __popc(b);
        __syncthreads();
        int before = running;
        for (int w = 0; w < warp; ++w) before += wsum[w];
        if (hit) {
            const int at = (padded ? tile0 * tm : start) + before + __popc(b & ((1u << lane) - 1u));
            sorted[at] = p;
            if (pos) pos[p] = at;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int w = 0; w < n_warps; ++w) tot += wsum[w];
            running += tot;
        }
        __syncthreads();
    }
    const int n_mine = (mine + tm - 1) / tm;
    for (int i = threadIdx.x; i < n_mine; i += blockDim.x) {
        if (tile0 + i >= max_tiles) break;
        tiles[(tile0 + i) * 3 + 0] = e;
        tiles[(tile0 + i) * 3 + 1] = (padded ? tile0 * tm : start) + i * tm;
        tiles[(tile0 + i) * 3 + 2] = min(tm, mine - i * tm);
        if (tab_up) { tab_up[tile0 + i] = e * up_rows; tab_down[tile0 + i] = e * down_rows; }
    }
    if (e == E - 1)
        for (int i = tile0 + n_mine + threadIdx.x; i < max_tiles; i += blockDim.x) {
            tiles[i * 3] = -1;
            if (tab_up) { tab_up[i] = -1; tab_down[i] = -1; }
        }
}

SP_API int sp_moe_tile_rows() { return ME_TM; }          // the smallest tile any path uses: sizes the tile table

static int moe_plan(const int* ids, int n_pairs, int E, int* counts, int* sorted, int* tiles, int max_tiles, int tm,
                    cudaStream_t stream) {
    moe_count_kernel<<<E, 256, 0, stream>>>(ids, n_pairs, counts);
    SP_CHECK_LAUNCH("moe_count");
    moe_place_kernel<<<E, n_pairs >= 2048 ? 1024 : 256, 0, stream>>>(ids, n_pairs, counts, E, sorted, tiles, max_tiles, tm, 0, nullptr, nullptr, nullptr, 0, 0);
    SP_CHECK_LAUNCH("moe_place");
    return 0;
}

// The plan for products that take whole 128-row tiles of one expert (the tcgen05 tile kernel's grouped form), and the
// rows in that order: sorted [max_tiles·128] (holes -1), pos [n_pairs], tab_up / tab_down [max_tiles], xs [max_tiles·128][W].
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted,
                                       __nv_bfloat16* __restrict__ xs, int rows, int top, int W) {
    const int per = W / 8;                                       // 16-byte pieces of a row
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)rows * per; i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / per), c = (int)(i % per);
        const int p = sorted[r];
        ((uint4*)xs)[i] = p >= 0 ? ((const uint4*)(x + (size_t)(p / top) * W))[c] : make_uint4(0, 0, 0, 0);
    }
}

SP_API int sp_moe_plan_tiles(const void* x, const int* ids, int T, int top, int W, int E, int up_rows, int down_rows, int* counts,
                             int* sorted, int* pos, int* tiles, int* tab_up, int* tab_down, int max_tiles, void* xs,
                             cudaStream_t stream) {
    const int n_pairs = T * top;
    if (n_pairs <= 0) return 0;
    if (W % 8 || (((uintptr_t)x | (uintptr_t)xs) & 15)) SP_FAIL("moe_plan_tiles: rows of %d do not move in 16-byte pieces", W);
    if ((n_pairs + 127) / 128 + E > max_tiles) SP_FAIL("moe_plan_tiles: the tile table is too short");
    SP_CHECK_CALL("moe_plan_tiles", cudaMemsetAsync(sorted, 0xff, (size_t)max_tiles * 128 * sizeof(int), stream));
    moe_count_kernel<<<E, 256, 0, stream>>>(ids, n_pairs, counts);
    SP_CHECK_LAUNCH("moe_count");
    moe_place_kernel<<<E, n_pairs >= 2048 ? 1024 : 256, 0, stream>>>(ids, n_pairs, counts, E, sorted, tiles, max_tiles, 128, 1, pos, tab_up, tab_down, up_rows, down_rows);
    SP_CHECK_LAUNCH("moe_place");
    const size_t n = (size_t)max_tiles * 128 * (W / 8);
    const size_t want = (n + 255) / 256;
    moe_gather_rows_kernel<<<(unsigned)(want > 148 * 16 ? 148 * 16 : want), 256, 0, stream>>>(
        (const __nv_bfloat16*)x, sorted, (__nv_bfloat16*)xs, max_tiles * 128, top, W);
    SP_CHECK_LAUNCH("moe_gather_rows");
    return 0;
}

// y[t] += Σ_k weight[t·top + k] · rows[pos[t·top + k]] in the order of k
__global__ void moe_combine_rows_kernel(const float* __restrict__ rows, const int* __restrict__ pos, const float* __restrict__ wts,
                                        float* __restrict__ y, size_t T, int top, int W) {
    const size_t n = T * (size_t)(W / 4);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / (W / 4);
        const int c = (int)(i % (W / 4));
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int k = 0; k < top; ++k) {
            const float wt = wts[t * top + k];
            const float4 r = ((const float4*)(rows + (size_t)pos[t * top + k] * W))[c];
            v.x += r.x * wt; v.y += r.y * wt; v.z += r.z * wt; v.w += r.w * wt;
        }
        float4 o = ((float4*)(y + t * W))[c];
        o.x += v.x; o.y += v.y; o.z += v.z; o.w += v.w;
        ((float4*)(y + t * W))[c] = o;
    }
}

SP_API int sp_moe_combine_rows(const float* rows, const int* pos, const float* wts, float* y, int T, int top, int W,
                               cudaStream_t stream) {
    if (T <= 0) return 0;
    if (W % 4 || (((uintptr_t)rows | (uintptr_t)y) & 15)) SP_FAIL("moe_combine_rows: rows of %d do not move in 16-byte pieces", W);
    const size_t n = (size_t)T * (W / 4);
    const size_t want = (n + 255) / 256;
    moe_combine_rows_kernel<<<(unsigned)(want > 148 * 16 ? 148 * 16 : want), 256, 0, stream>>>(rows, pos, wts, y, (size_t)T, top, W);
    SP_CHECK_LAUNCH("moe_combine_rows");
    return 0;
}

// FFMA tiles: ME_TM rows x ME_BN columns, K in blocks of ME_BK; thread (ty, tx) owns rows 2ty, 2ty+1 and columns
// 4tx … 4tx+3. Every output adds its products in the order of k, whatever tile it falls into.
#define ME_BN 64
#define ME_BK 32
template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
moe_up_kernel(const TA* __restrict__ x, const TW* __restrict__ wgu, const int* __restrict__ sorted,
              const int* __restrict__ tiles, TA* __restrict__ act, int top, int W, int F, float limit, float slope) {
    __shared__ float As[ME_BK][ME_TM + 1];
    __shared__ __align__(16) float Bg[ME_BK][ME_BN], Bu[ME_BK][ME_BN];
    __shared__ int tok[ME_TM];
    const int e = tiles[blockIdx.x * 3];
    if (e < 0) return;
    const int first = tiles[blockIdx.x * 3 + 1], rows = tiles[blockIdx.x * 3 + 2];
    const int n0 = blockIdx.y * ME_BN;
    if (threadIdx.x < ME_TM) tok[threadIdx.x] = threadIdx.x < rows ? sorted[first + threadIdx.x] / top : -1;
    __syncthreads();
    const TW* wg = wgu + (size_t)e * 2 * F * W;
    const TW* wu = wg + (size_t)F * W;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float ag[2][4] = {}, au[2][4] = {};
    for (int k0 = 0; k0 < W; k0 += ME_BK) {
        {
            const int m = threadIdx.x >> 3, kk = (threadIdx.x & 7) * 4;
            const int t = tok[m];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                As[kk + u][m] = (t >= 0 && k0 + kk + u < W) ? sp_ld(x, (size_t)t * W + k0 + kk + u) : 0.0f;
            const int n = threadIdx.x >> 2, k8 = (threadIdx.x & 3) * 8;
            const bool in = n0 + n < F;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool ok = in && k0 + k8 + u < W;
                Bg[k8 + u][n] = ok ? sp_ld(wg, (size_t)(n0 + n) * W + k0 + k8 + u) : 0.0f;
                Bu[k8 + u][n] = ok ? sp_ld(wu, (size_t)(n0 + n) * W + k0 + k8 + u) : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < ME_BK; ++k) {
            const float a0 = As[k][2 * ty], a1 = As[k][2 * ty + 1];
            const float4 g4 = *(const float4*)&Bg[k][4 * tx];
            const float4 u4 = *(const float4*)&Bu[k][4 * tx];
            const float g[4] = {g4.x, g4.y, g4.z, g4.w}, uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                ag[0][c] = fmaf(a0, g[c], ag[0][c]); ag[1][c] = fmaf(a1, g[c], ag[1][c]);
                au[0][c] = fmaf(a0, uu[c], au[0][c]); au[1][c] = fmaf(a1, uu[c], au[1][c]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int m = 2 * ty + r;
        if (m >= rows) continue;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int n = n0 + 4 * tx + c;
            if (n < F) sp_st(act, (size_t)(first + m) * F + n, hy_clamped_glu(ag[r][c], au[r][c], limit, slope));
        }
    }
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
moe_down_kernel(const TA* __restrict__ act, const TW* __restrict__ wd, const int* __restrict__ sorted,
                const int* __restrict__ tiles, const float* __restrict__ wts, float* __restrict__ out, int W, int F) {
    __shared__ float As[ME_BK][ME_TM + 1];
    __shared__ __align__(16) float Bs[ME_BK][ME_BN];
    const int e = tiles[blockIdx.x * 3];
    if (e < 0) return;
    const int first = tiles[blockIdx.x * 3 + 1], rows = tiles[blockIdx.x * 3 + 2];
    const int n0 = blockIdx.y * ME_BN;
    const TW* w = wd + (size_t)e * W * F;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < F; k0 += ME_BK) {
        {
            const int m = threadIdx.x >> 3, kk = (threadIdx.x & 7) * 4;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                As[kk + u][m] = (m < rows && k0 + kk + u < F) ? sp_ld(act, (size_t)(first + m) * F + k0 + kk + u) : 0.0f;
            const int n = threadIdx.x >> 2, k8 = (threadIdx.x & 3) * 8;
            const bool in = n0 + n < W;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                Bs[k8 + u][n] = (in && k0 + k8 + u < F) ? sp_ld(w, (size_t)(n0 + n) * F + k0 + k8 + u) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < ME_BK; ++k) {
            const float a0 = As[k][2 * ty], a1 = As[k][2 * ty + 1];
            const float4 b4 = *(const float4*)&Bs[k][4 * tx];
            const float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                acc[0][c] = fmaf(a0, b[c], acc[0][c]);
                acc[1][c] = fmaf(a1, b[c], acc[1][c]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int m = 2 * ty + r;
        if (m >= rows) continue;
        const int p = sorted[first + m];
        const float wt = wts[p];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int n = n0 + 4 * tx + c;
            if (n < W) out[(size_t)p * W + n] = acc[r][c] * wt;
        }
    }
}

// The same products on the tensor cores (bfloat16 operands, 32-bit accumulators): tiles of 128 rows x 64 columns, K in
// blocks of 32 through three shared-memory stages filled by cp.async (two in flight while one is multiplied: a decode
// step's tiles are bound by how many bytes a CTA has asked for); four warps, each 32 rows x all columns with
// mma.sync m16n8k16 (A and B fragments by ldmatrix from rows padded to 80 bytes); a group of 16 rows beyond the tile's
// rows (a decode step's tiles hold a row or two) is skipped. GLU: the tile holds the gate and the
// up columns of the same outputs and stores the activation; else the result times the pair's weight goes to the
// pair's row of ``out``. A row's sum runs over k in the same order whatever tile or batch the row is in.
#define MM_TM 128
#define MM_BN 64
#define MM_BK 32
#define MM_ROW 40
#define MM_STAGES 3
template <bool GLU>
constexpr size_t mm_smem_bytes() { return (size_t)MM_STAGES * (MM_TM + (GLU ? 2 : 1) * MM_BN) * MM_ROW * sizeof(__nv_bfloat16); }
template <bool GLU>
__global__ void __launch_bounds__(128, 3)
moe_mma_kernel(const __nv_bfloat16* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ Wt, long long w_stride,
               int N, int K, const int* __restrict__ sorted, const int* __restrict__ tiles, int top,
               __nv_bfloat16* __restrict__ act, float* __restrict__ out, const float* __restrict__ wts, float limit,
               float slope, int blk) {
    // ``blk`` (GLU): 0 = an expert's N gate rows, then its N up rows; else blocks of ``blk`` gate rows, each followed by
    // the ``blk`` up rows of the same outputs (the layout the tcgen05 tile kernel's gated epilogue reads)
    extern __shared__ __align__(16) unsigned char mm_smem[];
    typedef __nv_bfloat16 (*ATile)[MM_TM][MM_ROW];
    typedef __nv_bfloat16 (*BTile)[GLU ? 2 : 1][MM_BN][MM_ROW];
    ATile As = (ATile)mm_smem;                                                              // [stages][rows][k]
    BTile Bs = (BTile)(mm_smem + (size_t)MM_STAGES * MM_TM * MM_ROW * sizeof(__nv_bfloat16));   // [stages][gate / up][columns][k]
    __shared__ int src_row[MM_TM];
    const int e = tiles[blockIdx.x * 3];
    if (e < 0) return;
    const int first = tiles[blockIdx.x * 3 + 1], rows = tiles[blockIdx.x * 3 + 2];
    const int n0 = blockIdx.y * MM_BN;
    if (threadIdx.x < MM_TM) {
        const int m = (int)threadIdx.x;
        src_row[m] = m < rows ? (GLU ? sorted[first + m] / top : first + m) : -1;
    }
    __syncthreads();
    const __nv_bfloat16* w0 = Wt + (size_t)e * w_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nk = (K + MM_BK - 1) / MM_BK;

    // a thread's 16-byte pieces of the two tiles are the same in every block of K: their rows' addresses are found once
    constexpr int A_PIECES = MM_TM * 4 / 128, B_PIECES = (GLU ? 2 : 1) * MM_BN * 4 / 128;
    int a_src[A_PIECES], b_src[B_PIECES];             // element offsets from A and from the expert's weights; -1: zeros
#pragma unroll
    for (int i = 0; i < A_PIECES; ++i) {
        const int c = threadIdx.x + i * 128, src = src_row[c >> 2];
        a_src[i] = src >= 0 ? src * lda + (c & 3) * 8 : -1;
    }
#pragma unroll
    for (int i = 0; i < B_PIECES; ++i) {
        const int c = threadIdx.x + i * 128, m = c / (MM_BN * 4), n = n0 + ((c >> 2) % MM_BN);
        const int w_row = blk ? (n / blk) * 2 * blk + n % blk + m * blk : m * N + n;
        b_src[i] = n < N ? w_row * K + (c & 3) * 8 : -1;
    }
    const int a_rows = (rows + 15) / 16 * 16;
    auto load = [&](int kb, int st) {
#pragma unroll
        for (int i = 0; i < A_PIECES; ++i) {
            if (32 * i >= a_rows) break;                       // groups of rows that no product reads stay as they are
            const int c = threadIdx.x + i * 128, k = kb * MM_BK + (c & 3) * 8;
            if (a_src[i] >= 0 && k < K) cp_async16(smem_u32(&As[st][c >> 2][(c & 3) * 8]), A + a_src[i] + kb * MM_BK);
            else *(uint4*)&As[st][c >> 2][(c & 3) * 8] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < B_PIECES; ++i) {
            const int c = threadIdx.x + i * 128, k = kb * MM_BK + (c & 3) * 8;
            if (b_src[i] >= 0 && k < K) cp_async16(smem_u32(&Bs[st][c / (MM_BN * 4)][(c >> 2) % MM_BN][(c & 3) * 8]), w0 + b_src[i] + kb * MM_BK);
            else *(uint4*)&Bs[st][c / (MM_BN * 4)][(c >> 2) % MM_BN][(c & 3) * 8] = make_uint4(0, 0, 0, 0);
        }
        cp_async_commit();
    };

    float acc[2][GLU ? 2 : 1][8][4] = {};
    const bool live[2] = {warp * 32 < rows, warp * 32 + 16 < rows};
    const bool narrow = rows <= 16;
    load(0, 0);
    if (nk > 1) load(1, 1);
    for (int kb = 0; kb < nk; ++kb) {
        if (kb + 1 < nk) cp_async_wait<1>();          // block kb has landed; block kb + 1 may still be on its way
        else cp_async_wait<0>();
        __syncthreads();                                // ... for every thread's pieces, and block kb - 1 is done with
        if (kb + 2 < nk) load(kb + 2, (kb + 2) % MM_STAGES);
        const int st = kb % MM_STAGES;
        if (narrow) {
            // at most 16 rows (a decode step's tile): the four warps share the columns instead of the rows; warp w owns
            // column tiles 2w and 2w + 1 and keeps them in the accumulators' first two places
#pragma unroll
            for (int k16 = 0; k16 < MM_BK / 16; ++k16) {
                uint32_t a[4];
                ldmatrix_x4(smem_u32(&As[st][lane & 15][k16 * 16 + (lane >> 4) * 8]), a[0], a[1], a[2], a[3]);
#pragma unroll
                for (int m = 0; m < (GLU ? 2 : 1); ++m) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(smem_u32(&Bs[st][m][warp * 16 + (lane & 7) + (lane >> 4) * 8][k16 * 16 + ((lane >> 3) & 1) * 8]), b0, b1, b2, b3);
                    mma_bf16(acc[0][m][0], a, b0, b1);
                    mma_bf16(acc[0][m][1], a, b2, b3);
                }
            }
        } else if (live[0]) {
#pragma unroll
            for (int k16 = 0; k16 < MM_BK / 16; ++k16) {
                uint32_t a[2][4];
#pragma unroll
                for (int f = 0; f < 2; ++f)
                    if (f == 0 || live[1])
                        ldmatrix_x4(smem_u32(&As[st][warp * 32 + f * 16 + (lane & 15)][k16 * 16 + (lane >> 4) * 8]), a[f][0], a[f][1], a[f][2], a[f][3]);
#pragma unroll
                for (int m = 0; m < (GLU ? 2 : 1); ++m)
#pragma unroll
                    for (int np = 0; np < 4; ++np) {
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4(smem_u32(&Bs[st][m][np * 16 + (lane & 7) + (lane >> 4) * 8][k16 * 16 + ((lane >> 3) & 1) * 8]), b0, b1, b2, b3);
                        mma_bf16(acc[0][m][2 * np], a[0], b0, b1);
                        mma_bf16(acc[0][m][2 * np + 1], a[0], b2, b3);
                        if (live[1]) {
                            mma_bf16(acc[1][m][2 * np], a[1], b0, b1);
                            mma_bf16(acc[1][m][2 * np + 1], a[1], b2, b3);
                        }
                    }
            }
        }
    }
    if (narrow) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = (lane >> 2) + 8 * half;
            if (m >= rows) continue;
            const int p = GLU ? 0 : sorted[first + m];
            const float wt = GLU ? 0.0f : wts[p];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int n = n0 + (2 * warp + j) * 8 + (lane & 3) * 2;
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (n + u >= N) continue;
                    if (GLU) act[(size_t)(first + m) * N + n + u] = __float2bfloat16_rn(hy_clamped_glu(acc[0][0][j][2 * half + u], acc[0][GLU ? 1 : 0][j][2 * half + u], limit, slope));
                    else out[(size_t)p * N + n + u] = acc[0][0][j][2 * half + u] * wt;
                }
            }
        }
        return;
    }
#pragma unroll
    for (int f = 0; f < 2; ++f)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = warp * 32 + f * 16 + (lane >> 2) + 8 * half;
            if (m >= rows) continue;
            const int p = GLU ? 0 : sorted[first + m];
            const float wt = GLU ? 0.0f : wts[p];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const int n = n0 + nt * 8 + (lane & 3) * 2;
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (n + u >= N) continue;
                    if (GLU) act[(size_t)(first + m) * N + n + u] = __float2bfloat16_rn(hy_clamped_glu(acc[f][0][nt][2 * half + u], acc[f][GLU ? 1 : 0][nt][2 * half + u], limit, slope));
                    else out[(size_t)p * N + n + u] = acc[f][0][nt][2 * half + u] * wt;
                }
            }
        }
}

// y[t] += Σ_k out[t·top + k] in the order of k
__global__ void moe_combine_kernel(const float* __restrict__ out, float* __restrict__ y, size_t T, int top, int W) {
    const size_t n = T * (size_t)W;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / W;
        const int c = (int)(e % W);
        float v = 0.0f;
        for (int k = 0; k < top; ++k) v += out[(t * top + k) * W + c];
        y[e] += v;
    }
}

SP_API int sp_moe_experts(const void* x, int x_dt, const int* ids, const void* wgu, const void* wd, int w_dt, int E,
                          int* counts, int* sorted, int* tiles, int max_tiles, const float* wts, void* act, float* out_pairs,
                          float* y, int T, int top, int W, int F, float limit, float slope, int glu_block,
                          cudaStream_t stream) {
    if (T <= 0) return 0;
    const int n_pairs = T * top;
    if (glu_block && (x_dt != SP_DT_BF16 || w_dt != SP_DT_BF16 || F % glu_block))
        SP_FAIL("moe_experts: gate and up rows in blocks of %d are a bfloat16 layout for sizes that are multiples of it", glu_block);
    const bool mma = x_dt == SP_DT_BF16 && w_dt == SP_DT_BF16 && W % 8 == 0 && F % 8 == 0 &&
                     (((uintptr_t)x | (uintptr_t)wgu | (uintptr_t)wd | (uintptr_t)act) & 15) == 0;
    if (mma && ((long long)T * W >= (1LL << 31) || (long long)n_pairs * F >= (1LL << 31) || 2LL * F * W >= (1LL << 31)))
        SP_FAIL("moe_experts: operands beyond 2^31 elements");
    const int tm = mma ? MM_TM : ME_TM;
    if ((n_pairs + tm - 1) / tm + E > max_tiles) SP_FAIL("moe_experts: the tile table is too short");
    if (moe_plan(ids, n_pairs, E, counts, sorted, tiles, max_tiles, tm, stream)) return 1;
    if (mma) {
        const int used = (n_pairs + tm - 1) / tm + E;           // entries beyond the tiles in use say expert -1
        static SpPerDevice mma_ready;
        if (!mma_ready.done()) {
            if (cudaFuncSetAttribute(moe_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mm_smem_bytes<true>()) != cudaSuccess ||
                cudaFuncSetAttribute(moe_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mm_smem_bytes<false>()) != cudaSuccess)
                SP_FAIL("moe_experts: cannot raise the shared memory limit");
            mma_ready.mark();
        }
        moe_mma_kernel<true><<<dim3(used, (F + MM_BN - 1) / MM_BN), 128, mm_smem_bytes<true>(), stream>>>(
            (const __nv_bfloat16*)x, W, (const __nv_bfloat16*)wgu, 2LL * F * W, F, W, sorted, tiles, top,
            (__nv_bfloat16*)act, nullptr, nullptr, limit, slope, glu_block);
        SP_CHECK_LAUNCH("moe_up (tensor cores)");
        moe_mma_kernel<false><<<dim3(used, (W + MM_BN - 1) / MM_BN), 128, mm_smem_bytes<false>(), stream>>>(
            (const __nv_bfloat16*)act, F, (const __nv_bfloat16*)wd, (long long)W * F, W, F, sorted, tiles, top, nullptr,
            out_pairs, wts, 0.0f, 0.0f, 0);
        SP_CHECK_LAUNCH("moe_down (tensor cores)");
    } else {
        if (glu_block) SP_FAIL("moe_experts: sizes that the tensor-core tiles do not take need the plain layout of gate and up rows");
        const dim3 g_up(max_tiles, (F + ME_BN - 1) / ME_BN), g_down(max_tiles, (W + ME_BN - 1) / ME_BN);
#define ME_LAUNCH(TA, TW)                                                                                             \
    do {                                                                                                              \
        moe_up_kernel<TA, TW><<<g_up, 256, 0, stream>>>((const TA*)x, (const TW*)wgu, sorted, tiles, (TA*)act, top, W, F, limit, slope); \
        SP_CHECK_LAUNCH("moe_up");                                                                                    \
        moe_down_kernel<TA, TW><<<g_down, 256, 0, stream>>>((const TA*)act, (const TW*)wd, sorted, tiles, wts, out_pairs, W, F); \
        SP_CHECK_LAUNCH("moe_down");                                                                                  \
    } while (0)
        if (x_dt == SP_DT_F32 && w_dt == SP_DT_F32) ME_LAUNCH(float, float);
        else if (x_dt == SP_DT_BF16 && w_dt == SP_DT_BF16) ME_LAUNCH(__nv_bfloat16, __nv_bfloat16);
        else if (x_dt == SP_DT_F32 && w_dt == SP_DT_BF16) ME_LAUNCH(float, __nv_bfloat16);
        else SP_FAIL("moe_experts: unsupported dtype codes %d/%d", x_dt, w_dt);
#undef ME_LAUNCH
    }
    const size_t n = (size_t)T * W;
    const size_t want = (n + 255) / 256;
    moe_combine_kernel<<<(unsigned)(want > 148 * 16 ? 148 * 16 : want), 256, 0, stream>>>(out_pairs, y, (size_t)T, top, W);
    SP_CHECK_LAUNCH("moe_combine");
    return 0;
}
