// Small kernels of layers whose sublayers stand between two norms, and of gated attention mixers.
//
//   pair_embed          x_t = s · E[id_t] + B[(id_{t−1} · a + id_t · b) mod n]; the first token of a sequence takes the
//                       table's row n. The token before a step's first one is a word of per-slot state.
//   stream_norm_add     x ← x + r · y / sqrt(mean(y²) + eps) ⊙ w for a sublayer's output y (which is left zeroed for
//                       the next sublayer to add into); in the same pass the next reader's input: the norm of the new
//                       x with another weight, or the new x as it is, in the activation type
//   gated_qkv_store     a projected row [q | k | v | one gate per head]: biases, a query factor that grows with the
//                       logarithm of the position, rotation of neighbouring pairs over the first dims of every head,
//                       q out, k and v into their page rows, the gates out as 32-bit numbers
//   latent_rot_store    a projected row [q (per head: plain | rotated part) | low-rank row | shared key part | gates]:
//                       RMS norm of the low-rank row, rotation of the shared key part and of the queries' rotated
//                       parts, [normed row | rotated key part] into ONE page row, q and the gates out
//   gelu_gather_mul     out[t, j] = gelu_tanh(z[t, j]) · S[id_t, off + j]
//
// Norm statistics, angles (position · frequency, cosf / sinf), gates and sums are 32-bit; stores round to the
// activation type.
#include "common.cuh"

SP_API const char* sp_sandwich_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(sandwich)

// ============================================================== token row plus pair row
struct PairEmbedArgs {
    const void* table; const void* pairs; int dt;   // [vocab][W], [buckets + 1][W]
    const int* ids; const int* positions; const int* token_seq; const int* seq_start; const int* seq_slot;
    int* state; int n_slots;                        // [slots]: the last token of the step before
    float* out;
    int T, W, vocab, buckets, mul_prev, mul_cur;
    float scale;
    int* status;
};

__global__ void __launch_bounds__(128) pair_embed_kernel(PairEmbedArgs a) {
    __shared__ int row_s;
    const int t = blockIdx.x;
    if (t >= a.T) return;
    const int id = a.ids[t];
    const bool ok = id >= 0 && id < a.vocab;
    if (threadIdx.x == 0) {
        const int s = a.token_seq[t], first = a.seq_start[s];
        int slot = a.seq_slot[s];
        if (slot < 0 || slot >= a.n_slots) slot = 0;
        int row = a.buckets;                                        // a sequence's first token: the last row
        if (a.positions[t] > 0) {
            const int prev = t > first ? a.ids[t - 1] : a.state[slot];
            const long long mix = (long long)prev * a.mul_prev + (long long)id * a.mul_cur;
            row = (int)(((mix % a.buckets) + a.buckets) % a.buckets);
        }
        row_s = row;
        // the block of a sequence's first token of the step has read the state; it leaves the step's last token there
        if (t == first) a.state[slot] = a.ids[a.seq_start[s + 1] - 1];
        if (!ok && a.status) atomicCAS(a.status, 0, 301);           // a token id outside the table
    }
    __syncthreads();
    const int row = row_s;
    for (int c = threadIdx.x; c < a.W; c += blockDim.x) {
        const float e = ok ? sp_ld_dt(a.table, a.dt, (size_t)id * a.W + c) * a.scale : 0.0f;
        a.out[(size_t)t * a.W + c] = ok ? e + sp_ld_dt(a.pairs, a.dt, (size_t)row * a.W + c) : 0.0f;
    }
}

SP_API int sp_pair_embed(const void* table, const void* pairs, int dt, const int* ids, const int* positions,
                         const int* token_seq, const int* seq_start, const int* seq_slot, int* state, int n_slots, float* out,
                         int T, int W, int vocab, int buckets, int mul_prev, int mul_cur, float scale, int* status,
                         cudaStream_t stream) {
    if (T <= 0) return 0;
    if (buckets <= 0) SP_FAIL("pair_embed: the pair table needs at least one bucket, got %d", buckets);
    PairEmbedArgs a{table, pairs, dt, ids, positions, token_seq, seq_start, seq_slot, state, n_slots, out,
                    T, W, vocab, buckets, mul_prev, mul_cur, scale, status};
    pair_embed_kernel<<<T, 128, 0, stream>>>(a);
    SP_CHECK_LAUNCH("pair_embed");
    return 0;
}

// ============================================================== norm of a sublayer's output into the stream
struct NormAddArgs {
    float* x; float* y;                  // [T][W] the stream; the sublayer's output (zeroed on the way out)
    const float* w_post;                 // [W] weight of the output's norm, as it multiplies
    const float* w_next;                 // [W] weight of the next reader's norm, or null
    void* out; int out_dt;               // [T][W] the next reader's input, or null
    int next_mode;                       // 0: no output; 1: norm of the new x with w_next; 2: the new x as it is
    int T, W;
    float mult, eps;
};

template <int VEC>
__global__ void __launch_bounds__(256) stream_norm_add_kernel(NormAddArgs a) {
    __shared__ float red[32];
    sp_allow_dependents();
    sp_wait_for_predecessor();
    const int t = blockIdx.x;
    if (t >= a.T) return;
    float* xr = a.x + (size_t)t * a.W;
    float* yr = a.y + (size_t)t * a.W;
    float ss = 0.0f;
    if (VEC == 4) {
        for (int c = threadIdx.x * 4; c < a.W; c += blockDim.x * 4) {
            const float4 v = *(const float4*)(yr + c);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int c = threadIdx.x; c < a.W; c += blockDim.x) ss = fmaf(yr[c], yr[c], ss);
    }
    ss = sp_block_sum(ss, red);
    const float f = a.mult / sqrtf(ss / (float)a.W + a.eps);
    float s2 = 0.0f;
    if (VEC == 4) {
        for (int c = threadIdx.x * 4; c < a.W; c += blockDim.x * 4) {
            const float4 v = *(const float4*)(yr + c), w = *(const float4*)(a.w_post + c);
            float4 x = *(const float4*)(xr + c);
            x.x = fmaf(v.x * f, w.x, x.x); x.y = fmaf(v.y * f, w.y, x.y); x.z = fmaf(v.z * f, w.z, x.z); x.w = fmaf(v.w * f, w.w, x.w);
            *(float4*)(xr + c) = x;
            *(float4*)(yr + c) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            s2 = fmaf(x.x, x.x, s2); s2 = fmaf(x.y, x.y, s2); s2 = fmaf(x.z, x.z, s2); s2 = fmaf(x.w, x.w, s2);
        }
    } else {
        for (int c = threadIdx.x; c < a.W; c += blockDim.x) {
            const float x = fmaf(yr[c] * f, a.w_post[c], xr[c]);
            xr[c] = x;
            yr[c] = 0.0f;
            s2 = fmaf(x, x, s2);
        }
    }
    if (a.next_mode == 0) return;
    float g = 1.0f;
    if (a.next_mode == 1) {
        s2 = sp_block_sum(s2, red);
        g = 1.0f / sqrtf(s2 / (float)a.W + a.eps);
    }
    // every thread reads back the entries it wrote itself
    if (VEC == 4) {
        for (int c = threadIdx.x * 4; c < a.W; c += blockDim.x * 4) {
            float4 x = *(const float4*)(xr + c);
            if (a.next_mode == 1) {
                const float4 w = *(const float4*)(a.w_next + c);
                x.x *= g * w.x; x.y *= g * w.y; x.z *= g * w.z; x.w *= g * w.w;
            }
            if (a.out_dt == SP_DT_F32) {
                *(float4*)((float*)a.out + (size_t)t * a.W + c) = x;
            } else {
                __nv_bfloat162 p0 = __floats2bfloat162_rn(x.x, x.y), p1 = __floats2bfloat162_rn(x.z, x.w);
                uint2 pk;
                pk.x = *(uint32_t*)&p0; pk.y = *(uint32_t*)&p1;
                *(uint2*)((__nv_bfloat16*)a.out + (size_t)t * a.W + c) = pk;
            }
        }
    } else {
        for (int c = threadIdx.x; c < a.W; c += blockDim.x) {
            float x = xr[c];
            if (a.next_mode == 1) x *= g * a.w_next[c];
            sp_st_dt(a.out, a.out_dt, (size_t)t * a.W + c, x);
        }
    }
}

SP_API int sp_stream_norm_add(float* x, float* y, const float* w_post, const float* w_next, void* out, int out_dt,
                              int next_mode, int T, int W, float mult, float eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (next_mode < 0 || next_mode > 2 || (next_mode && !out) || (next_mode == 1 && !w_next))
        SP_FAIL("stream_norm_add: mode %d needs an output (and a weight for the norm)", next_mode);
    NormAddArgs a{x, y, w_post, w_next, out, out_dt, next_mode, T, W, mult, eps};
    const bool vec = (W % 4) == 0 && ((((uintptr_t)x | (uintptr_t)y | (uintptr_t)w_post | (uintptr_t)w_next | (uintptr_t)out) & 15) == 0);
    if (vec) SP_CHECK_CALL("stream_norm_add", sp_launch_dependent(stream_norm_add_kernel<4>, dim3(T), dim3(256), 0, stream, a));
    else SP_CHECK_CALL("stream_norm_add", sp_launch_dependent(stream_norm_add_kernel<1>, dim3(T), dim3(256), 0, stream, a));
    return 0;
}

// ============================================================== where a token's cached rows live
struct RowPlace {
    const int* token_seq; const int* positions; const int* seq_row; const int* page_table;
    int max_pages, page_size;
    SpRange rg;
};

__device__ __forceinline__ bool page_of(const RowPlace& pl, int t, int pos, int& page) {
    const int row = pl.seq_row[pl.token_seq[t]];
    if (!sp_index_ok(row, pl.rg.n_rows, pl.rg, 402) || !sp_index_ok(pos / pl.page_size, pl.max_pages, pl.rg, 403)) return false;
    page = pl.page_table[(size_t)row * pl.max_pages + pos / pl.page_size];
    return sp_index_ok(page, pl.rg.n_pages, pl.rg, 401);
}

// cos and sin of position · freq[i], times ``mult``, for i < half: cs[i], cs[half + i]
__device__ __forceinline__ void pair_angles(float* cs, const float* __restrict__ freq, int half, int pos, float mult) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * freq[i];
        cs[i] = cosf(ang) * mult;
        cs[half + i] = sinf(ang) * mult;
    }
}

// ============================================================== [q | k | v | gates]: bias, query factor, rotation, store
struct GatedQkvArgs {
    const float* proj; int ld;           // [T][ld] = [q: nh·d | k: nkv·d | v: nkv·vd | gates: nh]
    const void* bias; int b_dt;          // [nh·d + nkv·d + nkv·vd] or null
    void* q_out; int q_dt;               // [T][nh·d]
    void* kpool; void* vpool; int c_dt;  // [pages][nkv][page_size][d], [pages][nkv][page_size][vd]
    float* gates;                        // [T][nh] the gates' arguments (their sigmoid is taken where they multiply)
    const float* freq;                   // [rd/2] or null
    RowPlace pl;
    int T, nh, nkv, d, vd, rd, write_kv;
    float rot_mult;                      // multiplies cos and sin
    float temp_coef; int temp_every;     // q ← q · (1 + coef · ln(floor((pos + 1) / every) + 1)); coef 0: no factor
};

template <typename TO, typename TC>
__global__ void __launch_bounds__(128) gated_qkv_store_kernel(GatedQkvArgs a) {
    extern __shared__ float cs[];        // [2][rd/2]
    sp_allow_dependents();
    sp_wait_for_predecessor();
    const int t = blockIdx.x;
    if (t >= a.T) return;
    const int pos = a.pl.positions[t];
    const int half = a.rd >> 1;
    pair_angles(cs, a.freq, half, pos, a.rot_mult);
    __syncthreads();
    int page = 0;
    const bool place_ok = a.write_kv && page_of(a.pl, t, pos, page);
    const int off = pos % a.pl.page_size;
    const float* src = a.proj + (size_t)t * a.ld;
    const float temp = a.temp_coef != 0.0f
        ? 1.0f + a.temp_coef * logf((float)((pos + 1) / a.temp_every) + 1.0f) : 1.0f;       // the quotient of integers: exact
    TO* q_out = (TO*)a.q_out;
    TC* kpool = (TC*)a.kpool;
    TC* vpool = (TC*)a.vpool;
    const int d = a.d, nq = a.nh, nqk = a.nh + a.nkv;
    if ((d & 1) == 0) {
        const int dp = d >> 1;
        for (int e = threadIdx.x; e < nqk * dp; e += blockDim.x) {
            const int h = e / dp, i = e - h * dp;
            const int c = h * d + 2 * i;
            float u = src[c], v = src[c + 1];
            if (a.bias) { u += sp_ld_dt(a.bias, a.b_dt, c); v += sp_ld_dt(a.bias, a.b_dt, c + 1); }
            if (h < nq) { u *= temp; v *= temp; }
            if (2 * i < a.rd) {
                const float co = cs[i], si = cs[half + i];
                const float ru = u * co - v * si, rv = v * co + u * si;
                u = ru; v = rv;
            }
            if (h < nq) sp_st2(q_out, (size_t)t * nq * d + c, u, v);
            else if (place_ok) sp_st2(kpool, (((size_t)page * a.nkv + (h - nq)) * a.pl.page_size + off) * d + 2 * i, u, v);
        }
    } else {
        // an odd head size: element by element; rd is even, so the last dim never turns
        for (int e = threadIdx.x; e < nqk * d; e += blockDim.x) {
            const int h = e / d, i = e - h * d;
            float val = src[e] + (a.bias ? sp_ld_dt(a.bias, a.b_dt, e) : 0.0f);
            if (i < a.rd) {
                const int im = i ^ 1;
                const float other = src[h * d + im] + (a.bias ? sp_ld_dt(a.bias, a.b_dt, h * d + im) : 0.0f);
                const float co = cs[i >> 1], si = cs[half + (i >> 1)];
                val = (i & 1) ? val * co + other * si : val * co - other * si;
            }
            if (h < nq) sp_st(q_out, (size_t)t * nq * d + e, val * temp);
            else if (place_ok) sp_st(kpool, (((size_t)page * a.nkv + (h - nq)) * a.pl.page_size + off) * d + i, val);
        }
    }
    const int v0 = nqk * d;
    if (place_ok) {
        for (int e = threadIdx.x; e < a.nkv * a.vd; e += blockDim.x) {
            const int g = e / a.vd, r = e - g * a.vd;
            float v = src[v0 + e];
            if (a.bias) v += sp_ld_dt(a.bias, a.b_dt, v0 + e);
            sp_st(vpool, (((size_t)page * a.nkv + g) * a.pl.page_size + off) * a.vd + r, v);
        }
    }
    if (a.gates) {
        const int g0 = v0 + a.nkv * a.vd;
        for (int h = threadIdx.x; h < a.nh; h += blockDim.x) a.gates[(size_t)t * a.nh + h] = src[g0 + h];
    }
}

SP_API int sp_gated_qkv_store(const float* proj, int ld, const void* bias, int b_dt, void* q_out, int q_dt, void* kpool,
                              void* vpool, int c_dt, float* gates, const float* freq, const int* token_seq,
                              const int* positions, const int* seq_row, const int* page_table, int max_pages, int page_size,
                              int T, int nh, int nkv, int d, int vd, int rd, int write_kv, float rot_mult, float temp_coef,
                              int temp_every, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || vd <= 0 || rd < 0 || rd > d || (rd & 1)) SP_FAIL("gated_qkv_store: the rotated dims %d must be even and at most %d", rd, d);
    if (rd > 0 && !freq) SP_FAIL("gated_qkv_store: a frequency table is needed");
    if (temp_coef != 0.0f && temp_every <= 0) SP_FAIL("gated_qkv_store: the query factor's period must be positive, got %d", temp_every);
    if (ld < (nh + nkv) * d + nkv * vd + (gates ? nh : 0)) SP_FAIL("gated_qkv_store: rows of %d numbers are too short", ld);
    GatedQkvArgs a{proj, ld, bias, b_dt, q_out, q_dt, kpool, vpool, c_dt, gates, freq,
                   RowPlace{token_seq, positions, seq_row, page_table, max_pages, page_size, sp_range_host},
                   T, nh, nkv, d, vd, rd, write_kv, rot_mult, temp_coef, temp_every};
    const size_t smem = (size_t)(rd > 0 ? rd : 2) * sizeof(float);
#define GQ_LAUNCH(TO, TC) SP_CHECK_CALL("gated_qkv_store", sp_launch_dependent(gated_qkv_store_kernel<TO, TC>, dim3(T), dim3(128), smem, stream, a))
    if (q_dt == SP_DT_F32 && c_dt == SP_DT_F32) GQ_LAUNCH(float, float);
    else if (q_dt == SP_DT_BF16 && c_dt == SP_DT_BF16) GQ_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (q_dt == SP_DT_F32 && c_dt == SP_DT_BF16) GQ_LAUNCH(float, __nv_bfloat16);
    else if (q_dt == SP_DT_BF16 && c_dt == SP_DT_F32) GQ_LAUNCH(__nv_bfloat16, float);
    else SP_FAIL("gated_qkv_store: unsupported dtype codes %d/%d", q_dt, c_dt);
#undef GQ_LAUNCH
    return 0;
}

// ============================================================== [q | low-rank row | shared key part | gates]
struct LatentRotArgs {
    const float* proj; int ld;           // [T][ld] = [q: H·(d + rd) | row: rank | key part: rd | gates: H]; a reader has no row and no key part
    const void* wc; int w_dt;            // [rank] weight of the row's norm
    void* q_out; int q_dt;               // [T][H·(d + rd)], the rotated part of every head turned
    void* pool; int c_dt;                // [pages][page_size][rank + rd], or null (a reader)
    void* rows;                          // [T][rank + rd] like q_out, or null: the same rows token by token
    float* gates;                        // [T][H]
    const float* freq;                   // [rd/2]
    RowPlace pl;
    int T, H, d, rd, rank;
    float rot_mult, eps;
};

__global__ void __launch_bounds__(256) latent_rot_store_kernel(LatentRotArgs a) {
    extern __shared__ float cs[];        // [2][rd/2]
    __shared__ float red[32];
    sp_allow_dependents();
    sp_wait_for_predecessor();
    const int t = blockIdx.x;
    if (t >= a.T) return;
    const int pos = a.pl.positions[t];
    const int half = a.rd >> 1;
    pair_angles(cs, a.freq, half, pos, a.rot_mult);
    __syncthreads();
    const float* src = a.proj + (size_t)t * a.ld;
    const int qd = a.d + a.rd, nq = a.H * qd;
    // queries: the plain part passes, the rotated part turns pair by pair
    for (int e = threadIdx.x; e < a.H * a.d; e += blockDim.x) {
        const int h = e / a.d, i = e - h * a.d;
        sp_st_dt(a.q_out, a.q_dt, (size_t)t * nq + (size_t)h * qd + i, src[h * qd + i]);
    }
    for (int e = threadIdx.x; e < a.H * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        const int c = h * qd + a.d + 2 * i;
        const float u = src[c], v = src[c + 1], co = cs[i], si = cs[half + i];
        sp_st_dt(a.q_out, a.q_dt, (size_t)t * nq + c, u * co - v * si);
        sp_st_dt(a.q_out, a.q_dt, (size_t)t * nq + c + 1, v * co + u * si);
    }
    int g0 = nq;
    if (a.pool) {
        const float* lat = src + nq;
        float ss = 0.0f;
        for (int i = threadIdx.x; i < a.rank; i += blockDim.x) ss = fmaf(lat[i], lat[i], ss);
        ss = sp_block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)a.rank + a.eps);
        int page = 0;
        const bool place_ok = page_of(a.pl, t, pos, page);
        const int R = a.rank + a.rd;
        const size_t base = ((size_t)page * a.pl.page_size + pos % a.pl.page_size) * R;
        for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
            const float c = lat[i] * inv * sp_ld_dt(a.wc, a.w_dt, i);
            if (place_ok) sp_st_dt(a.pool, a.c_dt, base + i, c);
            if (a.rows) sp_st_dt(a.rows, a.q_dt, (size_t)t * R + i, c);
        }
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float u = lat[a.rank + 2 * i], v = lat[a.rank + 2 * i + 1], co = cs[i], si = cs[half + i];
            const float ru = u * co - v * si, rv = v * co + u * si;
            if (place_ok) {
                sp_st_dt(a.pool, a.c_dt, base + a.rank + 2 * i, ru);
                sp_st_dt(a.pool, a.c_dt, base + a.rank + 2 * i + 1, rv);
            }
            if (a.rows) {
                sp_st_dt(a.rows, a.q_dt, (size_t)t * R + a.rank + 2 * i, ru);
                sp_st_dt(a.rows, a.q_dt, (size_t)t * R + a.rank + 2 * i + 1, rv);
            }
        }
        g0 += R;
    }
    if (a.gates)
        for (int h = threadIdx.x; h < a.H; h += blockDim.x) a.gates[(size_t)t * a.H + h] = src[g0 + h];
}

SP_API int sp_latent_rot_store(const float* proj, int ld, const void* wc, int w_dt, void* q_out, int q_dt, void* pool, int c_dt,
                               void* rows, float* gates, const float* freq, const int* token_seq, const int* positions,
                               const int* seq_row, const int* page_table, int max_pages, int page_size, int T, int H, int d,
                               int rd, int rank, float rot_mult, float eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || d <= 0 || rank <= 0 || rd < 0 || (rd & 1)) SP_FAIL("latent_rot_store: sizes %d heads x (%d + %d), rank %d", H, d, rd, rank);
    if (rd > 0 && !freq) SP_FAIL("latent_rot_store: a frequency table is needed");
    if (ld < H * (d + rd) + (pool ? rank + rd : 0) + (gates ? H : 0)) SP_FAIL("latent_rot_store: rows of %d numbers are too short", ld);
    if (pool && !wc) SP_FAIL("latent_rot_store: the row's norm needs its weight");
    LatentRotArgs a{proj, ld, wc, w_dt, q_out, q_dt, pool, c_dt, rows, gates, freq,
                    RowPlace{token_seq, positions, seq_row, page_table, max_pages, page_size, sp_range_host},
                    T, H, d, rd, rank, rot_mult, eps};
    const size_t smem = (size_t)(rd > 0 ? rd : 2) * sizeof(float);
    SP_CHECK_CALL("latent_rot_store", sp_launch_dependent(latent_rot_store_kernel, dim3(T), dim3(256), smem, stream, a));
    return 0;
}

// ============================================================== gelu(z) times a gathered table row's part
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TZ, typename TW>
__global__ void gelu_gather_mul_kernel(const TZ* __restrict__ z, const TW* __restrict__ table, const int* __restrict__ ids,
                                       TZ* __restrict__ out, int T, int C, int ld, int off, int vocab) {
    const size_t n = (size_t)T * C;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(e / C), j = (int)(e - (size_t)t * C);
        const int id = ids[t];
        const float s = (id >= 0 && id < vocab) ? sp_ld(table, (size_t)id * ld + off + j) : 0.0f;
        sp_st(out, e, gelu_tanh_f(sp_ld(z, e)) * s);
    }
}

SP_API int sp_gelu_gather_mul(const void* z, int z_dt, const void* table, int t_dt, const int* ids, void* out, int T, int C,
                              int ld, int off, int vocab, cudaStream_t stream) {
    if (T <= 0 || C <= 0) return 0;
    if (off < 0 || off + C > ld) SP_FAIL("gelu_gather_mul: columns %d..%d lie outside rows of %d", off, off + C, ld);
    const size_t n = (size_t)T * C;
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
#define GG_LAUNCH(TZ, TW) gelu_gather_mul_kernel<TZ, TW><<<blocks, 256, 0, stream>>>((const TZ*)z, (const TW*)table, ids, (TZ*)out, T, C, ld, off, vocab)
    if (z_dt == SP_DT_F32 && t_dt == SP_DT_F32) GG_LAUNCH(float, float);
    else if (z_dt == SP_DT_BF16 && t_dt == SP_DT_BF16) GG_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (z_dt == SP_DT_F32 && t_dt == SP_DT_BF16) GG_LAUNCH(float, __nv_bfloat16);
    else if (z_dt == SP_DT_BF16 && t_dt == SP_DT_F32) GG_LAUNCH(__nv_bfloat16, float);
    else SP_FAIL("gelu_gather_mul: unsupported dtype codes %d/%d", z_dt, t_dt);
#undef GG_LAUNCH
    SP_CHECK_LAUNCH("gelu_gather_mul");
    return 0;
}
