// Attention through a cached low-rank latent.
//
// A token's keys and values of every head are linear images of one short row c (the latent), so only c is cached:
// one page row of ``rank`` numbers per token. The attention never expands keys or values:
//
//   score_h(i, j) = (U_k,hᵀ q_i,h) · c_j · scale          the query is carried into the latent's space once per token
//   out_i,h       = U_v,h (Σ_j p_h(i, j) c_j)             the weighted sum of latents is expanded once per token
//
//   latent_norm_store     RMS norms of the two halves of a projected row [q part | latent part]: the q part out in
//                         the activation type, the latent into its page row
//   headwise_product      out[t, h, :] = a[t, h, :] · W_h for a stack of small per-head matrices (either layout)
//   latent_attention      softmax over the visible latents with a sliding window and a per-head sink in the
//                         denominator; the page row serves as key and as value
//
// Norms, scores, softmax weights and all sums are 32-bit; stores round to the activation type. A row's reductions
// run in an order that depends on its own sequence only.
#include "common.cuh"

SP_API const char* sp_latent_last_error() { return sp_error_text; }
SP_DEFINE_RANGE_API(latent)

// ============================================================== norms of the projected row, latent to pages
struct LnArgs {
    const float* proj; int ld;                      // [T][ld] = [q part: qr | latent part: rank]
    const void* wq; const void* wc; int w_dt;       // norm weights [qr], [rank]
    void* cq; int cq_dt;                            // [T][qr]
    void* pool; int pool_dt;                        // [pages][page_size][rank], or null: the latent part is absent
    void* rows;                                     // [T][rank] like cq, or null: the same latents token by token
    const int* token_seq; const int* positions; const int* seq_row; const int* page_table; int max_pages, page_size;
    int T, qr, rank;
    float eps;
    SpRange rg;
};

__global__ void __launch_bounds__(256) latent_norm_store_kernel(LnArgs a) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    if (t >= a.T) return;
    const float* row = a.proj + (size_t)t * a.ld;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < a.qr; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    ss = sp_block_sum(ss, red);
    const float inv_q = 1.0f / sqrtf(ss / (float)a.qr + a.eps);
    for (int i = threadIdx.x; i < a.qr; i += blockDim.x)
        sp_st_dt(a.cq, a.cq_dt, (size_t)t * a.qr + i, row[i] * inv_q * sp_ld_dt(a.wq, a.w_dt, i));
    if (!a.pool) return;
    const float* lat = row + a.qr;
    float sc = 0.0f;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) sc = fmaf(lat[i], lat[i], sc);
    sc = sp_block_sum(sc, red);
    const float inv_c = 1.0f / sqrtf(sc / (float)a.rank + a.eps);
    const int s = a.token_seq[t], pos = a.positions[t];
    const int prow = a.seq_row[s];
    if (!sp_index_ok(prow, a.rg.n_rows, a.rg, 402) || !sp_index_ok(pos / a.page_size, a.max_pages, a.rg, 403)) return;
    const int page = a.page_table[(size_t)prow * a.max_pages + pos / a.page_size];
    if (!sp_index_ok(page, a.rg.n_pages, a.rg, 401)) return;
    const size_t base = ((size_t)page * a.page_size + pos % a.page_size) * a.rank;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
        const float c = lat[i] * inv_c * sp_ld_dt(a.wc, a.w_dt, i);
        sp_st_dt(a.pool, a.pool_dt, base + i, c);
        if (a.rows) sp_st_dt(a.rows, a.cq_dt, (size_t)t * a.rank + i, c);
    }
}

SP_API int sp_latent_norm_store(const float* proj, int ld, const void* wq, const void* wc, int w_dt, void* cq, int cq_dt,
                                void* pool, int pool_dt, const int* token_seq, const int* positions, const int* seq_row,
                                const int* page_table, int max_pages, int page_size, int T, int qr, int rank, float eps,
                                void* rows, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (qr <= 0 || rank <= 0 || ld < qr + (pool ? rank : 0)) SP_FAIL("latent_norm_store: parts of %d and %d do not fit rows of %d", qr, rank, ld);
    LnArgs a{proj, ld, wq, wc, w_dt, cq, cq_dt, pool, pool_dt, rows, token_seq, positions, seq_row, page_table, max_pages,
             page_size, T, qr, rank, eps, sp_range_host};
    latent_norm_store_kernel<<<T, 256, 0, stream>>>(a);
    SP_CHECK_LAUNCH("latent_norm_store");
    return 0;
}

// ============================================================== a stack of small matrices, one per head
// out[t][h][n] = Σ_k a[t][h][k] · W_h[k][n]. ``w`` holds the heads' matrices one after another, either as rows of k
// (w[h][k][n], ``w_rows_are_k``) or as rows of n (w[h][n][k]): a slice [h·N … (h+1)·N) of rows of a matrix stored
// [out, in]. A block takes HW_TT tokens x HW_TN outputs of one head; a and W pass through shared memory in blocks
// of HW_TK of k; a thread owns one output column for all the block's tokens and adds over k in ascending order
// (so a token's result does not depend on the block it falls into, nor on HW_TT). Steps of a few tokens (decoding)
// take blocks of 8 tokens: a quarter of the multiply-adds, which are all that such a block waits for.
#define HW_TN 128
#define HW_TK 32
template <typename TA, typename TW, typename TO, int HW_TT>
__global__ void __launch_bounds__(HW_TN)
headwise_product_kernel(const TA* __restrict__ a, const TW* __restrict__ w, TO* __restrict__ out, int T, int H, int K, int N,
                        int w_rows_are_k) {
    __shared__ float As[HW_TT][HW_TK + 1];
    __shared__ float Ws[HW_TK][HW_TN + 1];
    const int h = blockIdx.y, t0 = blockIdx.x * HW_TT, n0 = blockIdx.z * HW_TN;
    const int tid = threadIdx.x;
    float acc[HW_TT];
#pragma unroll
    for (int i = 0; i < HW_TT; ++i) acc[i] = 0.0f;
    const TW* wh = w + (size_t)h * K * N;
    for (int k0 = 0; k0 < K; k0 += HW_TK) {
        for (int e = tid; e < HW_TT * HW_TK; e += HW_TN) {
            const int tt = e / HW_TK, kk = e % HW_TK;
            const int t = t0 + tt, k = k0 + kk;
            As[tt][kk] = (t < T && k < K) ? sp_ld(a, ((size_t)t * H + h) * K + k) : 0.0f;
        }
        if (w_rows_are_k) {
#pragma unroll 16
            for (int e = tid; e < HW_TK * HW_TN; e += HW_TN) {
                const int kk = e / HW_TN, nn = e % HW_TN;
                const int k = k0 + kk, n = n0 + nn;
                Ws[kk][nn] = (k < K && n < N) ? sp_ld(wh, (size_t)k * N + n) : 0.0f;
            }
        } else {
#pragma unroll 16
            for (int e = tid; e < HW_TK * HW_TN; e += HW_TN) {
                const int nn = e / HW_TK, kk = e % HW_TK;
                const int k = k0 + kk, n = n0 + nn;
                Ws[kk][nn] = (k < K && n < N) ? sp_ld(wh, (size_t)n * K + k) : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll 4
        for (int kk = 0; kk < HW_TK; ++kk) {
            const float wv = Ws[kk][tid];
#pragma unroll
            for (int i = 0; i < HW_TT; ++i) acc[i] = fmaf(As[i][kk], wv, acc[i]);
        }
        __syncthreads();
    }
    const int n = n0 + tid;
    if (n >= N) return;
#pragma unroll
    for (int i = 0; i < HW_TT; ++i) {
        const int t = t0 + i;
        if (t < T) sp_st(out, ((size_t)t * H + h) * N + n, acc[i]);
    }
}

// The same for a few tokens (a decode step), where the weights' bytes are all there is to do: a warp per output
// row n of W_h stored [n][k], its lanes striding over k in pairs of bfloat16, the tokens' inputs of this head waiting
// in shared memory as 32-bit; a lane adds its k in ascending order, the lanes' sums meet by shuffles. HS_ROWS output rows
// per block keep every SM busy on a stack of a megabyte.
#define HS_TMAX 16
#define HS_ROWS 32
template <typename TA, typename TO>
__global__ void __launch_bounds__(256)
headwise_small_kernel(const TA* __restrict__ a, const __nv_bfloat16* __restrict__ w, TO* __restrict__ out, int T, int H, int K, int N) {
    extern __shared__ float hs_a[];                           // [T][K]
    const int h = blockIdx.x, n0 = blockIdx.y * HS_ROWS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = threadIdx.x; e < T * K; e += 256) {
        const int t = e / K, k = e % K;
        hs_a[e] = sp_ld(a, ((size_t)t * H + h) * K + k);
    }
    __syncthreads();
    const __nv_bfloat16* wh = w + (size_t)h * N * K;
    for (int n = n0 + warp; n < min(N, n0 + HS_ROWS); n += 8) {
        const __nv_bfloat162* row = (const __nv_bfloat162*)(wh + (size_t)n * K);
        float acc[HS_TMAX];
#pragma unroll
        for (int t = 0; t < HS_TMAX; ++t) acc[t] = 0.0f;
#pragma unroll 4
        for (int k2 = lane; k2 < K / 2; k2 += 32) {
            const float2 wv = __bfloat1622float2(row[k2]);
#pragma unroll
            for (int t = 0; t < HS_TMAX; ++t)
                if (t < T) {
                    const float2 av = *(const float2*)(hs_a + t * K + 2 * k2);
                    acc[t] = fmaf(av.y, wv.y, fmaf(av.x, wv.x, acc[t]));
                }
        }
#pragma unroll
        for (int t = 0; t < HS_TMAX; ++t)
            if (t < T) {
                float v = acc[t];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) sp_st(out, ((size_t)t * H + h) * N + n, v);
            }
    }
}

SP_API int sp_headwise_product(const void* a, int a_dt, const void* w, int w_dt, void* out, int out_dt, int T, int H, int K,
                               int N, int w_rows_are_k, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || K <= 0 || N <= 0) SP_FAIL("headwise_product: sizes %d x %d x %d", H, K, N);
    if (T <= HS_TMAX && !w_rows_are_k && w_dt == SP_DT_BF16 && K % 2 == 0 && (size_t)T * K * 4 <= 48 * 1024 && H <= 65535 &&
        (a_dt == SP_DT_BF16 || a_dt == SP_DT_F32) && a_dt == out_dt && ((uintptr_t)w & 3) == 0) {
        const dim3 grid(H, (N + HS_ROWS - 1) / HS_ROWS);
        const size_t smem = (size_t)T * K * 4;
        if (a_dt == SP_DT_BF16)
            headwise_small_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, smem, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, T, H, K, N);
        else
            headwise_small_kernel<float, float><<<grid, 256, smem, stream>>>((const float*)a, (const __nv_bfloat16*)w, (float*)out, T, H, K, N);
        SP_CHECK_LAUNCH("headwise_small");
        return 0;
    }
    const int tt = T <= 16 ? 8 : 32;
    const dim3 grid((T + tt - 1) / tt, H, (N + HW_TN - 1) / HW_TN);
    if (grid.y > 65535 || grid.z > 65535) SP_FAIL("headwise_product: %d heads or %d outputs are too many for one launch", H, N);
#define HW_LAUNCH(TA, TW, TO)                                                                                                  \
    do {                                                                                                                       \
        if (tt == 8) headwise_product_kernel<TA, TW, TO, 8><<<grid, HW_TN, 0, stream>>>((const TA*)a, (const TW*)w, (TO*)out, T, H, K, N, w_rows_are_k); \
        else headwise_product_kernel<TA, TW, TO, 32><<<grid, HW_TN, 0, stream>>>((const TA*)a, (const TW*)w, (TO*)out, T, H, K, N, w_rows_are_k); \
    } while (0)
    typedef __nv_bfloat16 bf;
    if (a_dt == SP_DT_F32 && w_dt == SP_DT_F32 && out_dt == SP_DT_F32) HW_LAUNCH(float, float, float);
    else if (a_dt == SP_DT_BF16 && w_dt == SP_DT_BF16 && out_dt == SP_DT_BF16) HW_LAUNCH(bf, bf, bf);
    else if (a_dt == SP_DT_BF16 && w_dt == SP_DT_BF16 && out_dt == SP_DT_F32) HW_LAUNCH(bf, bf, float);
    else if (a_dt == SP_DT_F32 && w_dt == SP_DT_BF16 && out_dt == SP_DT_BF16) HW_LAUNCH(float, bf, bf);
    else if (a_dt == SP_DT_F32 && w_dt == SP_DT_BF16 && out_dt == SP_DT_F32) HW_LAUNCH(float, bf, float);
    else SP_FAIL("headwise_product: unsupported dtype codes %d/%d/%d", a_dt, w_dt, out_dt);
#undef HW_LAUNCH
    SP_CHECK_LAUNCH("headwise_product");
    return 0;
}

// ============================================================== the attention itself, on tensor cores
// Queries arrive in the latent's space: q [T][H][RANK] (bfloat16). All heads read the same page rows c_j, and a row
// is key and value at once, so a tile of LF_KEYS cached rows is fetched into shared memory ONCE and serves both
// products of a block of LF_ROWS query rows:
//
//   S = Q · Cᵀ            (LF_ROWS x LF_KEYS, contraction over RANK)      mma.sync m16n8k16, bfloat16 in, 32-bit out
//   P = online softmax(S · scale) in 32-bit, rounded to bfloat16 for the second product; the row sums add the rounded
//       weights, so numerator and denominator agree
//   O = O · rescale + P · C   (LF_ROWS x RANK, contraction over LF_KEYS)
//
// A block's rows are LF_ROWS consecutive tokens of one sequence for one head (a prompt's portion: grid = heads x
// token tiles) or up to LF_ROWS heads of one token (a decode step: grid = head groups x sequences). Eight warps: for S
// a warp owns 16 rows x 8 keys over all of RANK; for O it owns RANK/8 columns of all rows (the accumulators are the
// only large register array: 2 x RANK/64 x 4 floats per thread). Tiles of cached rows arrive by cp.async in two
// stages. A row sees key j when lo <= j <= its position (lo = position − window + 1 with a window, else 0); a sink
// adds e^{sink_h} to a row's denominator at the end. Keys are visited in ascending order whatever the block, so a
// row's sums do not depend on how the tokens were cut into steps beyond the rounding of the rescaling. A decode step
// has few rows and many keys: its visible keys are shared out over blockIdx.z (as many blocks as fill the SMs, at
// least 128 keys each), every share leaves its unnormalised sums with their (max, sum) in scratch, and a second
// kernel adds the shares in ascending order of keys and brings the sink in once.
#include "flash_common.cuh"

namespace {
constexpr int LF_ROWS = 32;
constexpr int LF_KEYS = 32;
constexpr int LF_PAGE = 64;

template <int RANK>
struct LfSmem {
    static constexpr int LD = RANK + 8;                       // elements per row: 16 bytes of padding spread the banks
    static constexpr int Q_BYTES = LF_ROWS * LD * 2;
    static constexpr int K_BYTES = LF_KEYS * LD * 2;
    static constexpr int S_LD = LF_KEYS + 1;
    static constexpr int S_BYTES = LF_ROWS * S_LD * 4;
    static constexpr int P_LD = LF_KEYS + 8;
    static constexpr int P_BYTES = LF_ROWS * P_LD * 2;
    static constexpr int META_BYTES = LF_ROWS * 4 * 6;        // rescale, max, sum, position, token, head per row
    static constexpr int OFF_K = Q_BYTES, OFF_S = OFF_K + 2 * K_BYTES, OFF_P = OFF_S + S_BYTES, OFF_META = OFF_P + P_BYTES;
    static constexpr int TOTAL = OFF_META + META_BYTES;
};

struct LfArgs {
    const __nv_bfloat16* q; __nv_bfloat16* out; const __nv_bfloat16* pool;
    const int* page_table; const int* seq_row; int max_pages;
    const int* seq_start; const int* positions; int n_seqs;
    const float* sink; int H, window; float scale_log2; int decode;
    SpRange rg;
    // a decode step's keys split over blockIdx.z: ``chunk_tiles`` key tiles per block, unnormalised partial sums
    // [sequence][head][chunk][RANK] and their (max, sum) pairs to scratch, combined by ``latent_combine_kernel``
    int n_chunks, chunk_tiles; float* part_o; float* part_ml;
};

template <int RANK>
__global__ void __launch_bounds__(256) latent_flash_kernel(LfArgs a) {
    using L = LfSmem<RANK>;
    constexpr int CPW = RANK / 8;                             // output columns per warp
    static_assert(RANK % 128 == 0, "a warp's columns come in pairs of 8-wide tiles");
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t q_s = smem_u32(smem), k_s = q_s + L::OFF_K, p_s = q_s + L::OFF_P;
    float* S = (float*)(smem + L::OFF_S);
    __nv_bfloat16* P = (__nv_bfloat16*)(smem + L::OFF_P);
    float* fac_s = (float*)(smem + L::OFF_META);
    float* m_s = fac_s + LF_ROWS;
    float* l_s = m_s + LF_ROWS;
    int* pos_s = (int*)(l_s + LF_ROWS);
    int* tok_s = pos_s + LF_ROWS;
    int* head_s = tok_s + LF_ROWS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- which rows
    int b = 0, min_pos = 0, max_pos = 0;
    if (a.decode) {
        b = blockIdx.y;
        const int t = a.seq_start[b], pos = a.positions[t];
        min_pos = max_pos = pos;
        if (tid < LF_ROWS) {
            const int h = blockIdx.x * LF_ROWS + tid;
            pos_s[tid] = h < a.H ? pos : -1;
            tok_s[tid] = t;
            head_s[tid] = h < a.H ? h : 0;
        }
    } else {
        int x = blockIdx.y, first = 0, n_new = 0;
        for (; b < a.n_seqs; ++b) {
            first = a.seq_start[b];
            n_new = a.seq_start[b + 1] - first;
            const int nt = (n_new + LF_ROWS - 1) / LF_ROWS;
            if (x < nt) break;
            x -= nt;
        }
        if (b >= a.n_seqs) return;
        const int t0 = first + x * LF_ROWS, n_rows = min(LF_ROWS, n_new - x * LF_ROWS);
        const int pos0 = a.positions[t0];
        min_pos = pos0;
        max_pos = pos0 + n_rows - 1;
        if (tid < LF_ROWS) {
            pos_s[tid] = tid < n_rows ? pos0 + tid : -1;
            tok_s[tid] = t0 + (tid < n_rows ? tid : 0);
            head_s[tid] = blockIdx.x;
        }
    }
    __syncthreads();
    const int* pt = a.page_table + (size_t)sp_checked_row(a.seq_row[b], a.rg) * a.max_pages;
    const int lo_key = (a.window > 0 && min_pos - a.window + 1 > 0) ? min_pos - a.window + 1 : 0;
    int j_lo = lo_key / LF_KEYS, j_hi = max_pos / LF_KEYS;
    const bool split = a.n_chunks > 1;
    if (split) {                                              // this block's share of the key tiles, counted from the first visible one
        j_lo += blockIdx.z * a.chunk_tiles;
        j_hi = min(j_hi, j_lo + a.chunk_tiles - 1);
        if (j_lo > j_hi) {                                    // beyond the row's keys: an empty share
            if (tid < LF_ROWS && pos_s[tid] >= 0) {
                float* ml = a.part_ml + (((size_t)b * a.H + head_s[tid]) * a.n_chunks + blockIdx.z) * 2;
                ml[0] = -INFINITY;
                ml[1] = 0.0f;
            }
            return;
        }
    }

    // ---- the queries, then the first tile of cached rows
    constexpr int CHUNKS = RANK / 8;                          // 16-byte pieces per row
    for (int c = tid; c < LF_ROWS * CHUNKS; c += 256) {
        const int r = c / CHUNKS, k = c % CHUNKS;
        const uint32_t d = q_s + (r * L::LD + k * 8) * 2;
        if (pos_s[r] >= 0) cp_async16(d, a.q + ((size_t)tok_s[r] * a.H + head_s[r]) * RANK + k * 8);
        else asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(d), "r"(0u) : "memory");
    }
    auto load_keys = [&](int jt, int stage) {
        const int j0 = jt * LF_KEYS;
        const int page = sp_checked_page(pt[sp_checked_entry(j0 / LF_PAGE, a.max_pages, a.rg)], a.rg);
        const __nv_bfloat16* src = a.pool + ((size_t)page * LF_PAGE + j0 % LF_PAGE) * RANK;
        const uint32_t dst = k_s + stage * L::K_BYTES;
        for (int c = tid; c < LF_KEYS * CHUNKS; c += 256) {
            const int r = c / CHUNKS, k = c % CHUNKS;
            cp_async16(dst + (r * L::LD + k * 8) * 2, src + (size_t)r * RANK + k * 8);
        }
    };
    load_keys(j_lo, 0);
    cp_async_commit();

    float o[2][CPW / 8][4];
#pragma unroll
    for (int rt = 0; rt < 2; ++rt)
#pragma unroll
        for (int nt = 0; nt < CPW / 8; ++nt) o[rt][nt][0] = o[rt][nt][1] = o[rt][nt][2] = o[rt][nt][3] = 0.0f;
    // the softmax's view: thread -> (row, four neighbouring keys of the tile); the row's eight threads are neighbours in a warp
    const int srow = tid >> 3, sub = tid & 7;
    const int spos = pos_s[srow];
    const int slo = a.window > 0 ? spos - a.window + 1 : 0;
    float m = -INFINITY, l = 0.0f;
    const int rt_s = warp & 1, kg = warp >> 1;                // the score product's view: 16 rows x 8 keys per warp

    for (int jt = j_lo; jt <= j_hi; ++jt) {
        const int stage = (jt - j_lo) & 1;
        if (jt < j_hi) load_keys(jt + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t kt = k_s + stage * L::K_BYTES;
        {   // S = Q · Cᵀ
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const uint32_t a_addr = q_s + ((rt_s * 16 + (lane & 15)) * L::LD + (lane >> 4) * 8) * 2;
            const uint32_t b_addr = kt + ((kg * 8 + (lane & 7)) * L::LD + (lane >> 3) * 8) * 2;
#pragma unroll 4
            for (int ks = 0; ks < RANK / 16; ks += 2) {
                uint32_t af[4], ag[4], b0, b1, b2, b3;
                ldmatrix_x4(a_addr + ks * 32, af[0], af[1], af[2], af[3]);
                ldmatrix_x4(a_addr + ks * 32 + 32, ag[0], ag[1], ag[2], ag[3]);
                ldmatrix_x4(b_addr + ks * 32, b0, b1, b2, b3);
                mma_bf16(acc, af, b0, b1);
                mma_bf16(acc, ag, b2, b3);
            }
            float* dst = S + (rt_s * 16 + (lane >> 2)) * L::S_LD + kg * 8 + 2 * (lane & 3);
            dst[0] = acc[0]; dst[1] = acc[1];
            dst[8 * L::S_LD] = acc[2]; dst[8 * L::S_LD + 1] = acc[3];
        }
        __syncthreads();
        {   // the online softmax of the tile's scores
            float s[4], tmax = -INFINITY;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j = jt * LF_KEYS + sub * 4 + i;
                const bool seen = spos >= 0 && j <= spos && j >= slo;
                s[i] = seen ? S[srow * L::S_LD + sub * 4 + i] * a.scale_log2 : -INFINITY;
                tmax = fmaxf(tmax, s[i]);
            }
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
            const float m_new = fmaxf(m, tmax);
            float fac = 1.0f, psum = 0.0f;
            __nv_bfloat16 pb[4];
            if (m_new == -INFINITY) {
#pragma unroll
                for (int i = 0; i < 4; ++i) pb[i] = __float2bfloat16_rn(0.0f);
            } else {
                fac = fast_exp2(m - m_new);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    pb[i] = __float2bfloat16_rn(fast_exp2(s[i] - m_new));
                    psum += __bfloat162float(pb[i]);
                }
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            psum += __shfl_xor_sync(0xffffffffu, psum, 4);
            l = l * fac + psum;
            m = m_new;
            __nv_bfloat162* pd = (__nv_bfloat162*)(P + srow * L::P_LD + sub * 4);
            pd[0] = __halves2bfloat162(pb[0], pb[1]);
            pd[1] = __halves2bfloat162(pb[2], pb[3]);
            if (sub == 0) fac_s[srow] = fac;
        }
        __syncthreads();
        {   // O = O · rescale + P · C
#pragma unroll
            for (int rt = 0; rt < 2; ++rt) {
                const float f0 = fac_s[rt * 16 + (lane >> 2)], f1 = fac_s[rt * 16 + (lane >> 2) + 8];
#pragma unroll
                for (int nt = 0; nt < CPW / 8; ++nt) { o[rt][nt][0] *= f0; o[rt][nt][1] *= f0; o[rt][nt][2] *= f1; o[rt][nt][3] *= f1; }
            }
#pragma unroll
            for (int ks = 0; ks < LF_KEYS / 16; ++ks) {
                uint32_t pa[2][4];
#pragma unroll
                for (int rt = 0; rt < 2; ++rt)
                    ldmatrix_x4(p_s + ((rt * 16 + (lane & 15)) * L::P_LD + ks * 16 + (lane >> 4) * 8) * 2, pa[rt][0], pa[rt][1], pa[rt][2], pa[rt][3]);
                const uint32_t v_addr = kt + ((ks * 16 + (lane & 15)) * L::LD + warp * CPW + (lane >> 4) * 8) * 2;
#pragma unroll
                for (int np = 0; np < CPW / 16; ++np) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(v_addr + np * 32, b0, b1, b2, b3);
#pragma unroll
                    for (int rt = 0; rt < 2; ++rt) {
                        mma_bf16(o[rt][2 * np], pa[rt], b0, b1);
                        mma_bf16(o[rt][2 * np + 1], pa[rt], b2, b3);
                    }
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if (sub == 0) { m_s[srow] = m; l_s[srow] = l; }
    __syncthreads();
    if (split) {
        if (tid < LF_ROWS && pos_s[tid] >= 0) {
            float* ml = a.part_ml + (((size_t)b * a.H + head_s[tid]) * a.n_chunks + blockIdx.z) * 2;
            ml[0] = m_s[tid];
            ml[1] = l_s[tid];
        }
#pragma unroll
        for (int rt = 0; rt < 2; ++rt)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int r = rt * 16 + (lane >> 2) + hf * 8;
                if (pos_s[r] < 0) continue;
                float* dst = a.part_o + (((size_t)b * a.H + head_s[r]) * a.n_chunks + blockIdx.z) * RANK + warp * CPW + 2 * (lane & 3);
#pragma unroll
                for (int nt = 0; nt < CPW / 8; ++nt)
                    *(float2*)(dst + nt * 8) = make_float2(o[rt][nt][2 * hf], o[rt][nt][2 * hf + 1]);
            }
        return;
    }
#pragma unroll
    for (int rt = 0; rt < 2; ++rt)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int r = rt * 16 + (lane >> 2) + hf * 8;
            if (pos_s[r] < 0) continue;
            const int h = head_s[r];
            float mr = m_s[r], lr = l_s[r], f = 1.0f;
            if (a.sink) {
                const float sk = a.sink[h] * LOG2E;
                const float m_all = fmaxf(mr, sk);
                f = fast_exp2(mr - m_all);
                lr = lr * f + fast_exp2(sk - m_all);
            }
            const float inv = f / lr;
            __nv_bfloat16* dst = a.out + ((size_t)tok_s[r] * a.H + h) * RANK + warp * CPW + 2 * (lane & 3);
#pragma unroll
            for (int nt = 0; nt < CPW / 8; ++nt)
                *(uint32_t*)(dst + nt * 8) = pack_bf16(o[rt][nt][2 * hf] * inv, o[rt][nt][2 * hf + 1] * inv);
        }
}

// The shares of one (sequence, head) in ascending order of keys: out = Σ_c O_c 2^{m_c − M} / (Σ_c l_c 2^{m_c − M} + 2^{sink − M}).
__global__ void __launch_bounds__(128) latent_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                             __nv_bfloat16* __restrict__ out, const int* __restrict__ seq_start,
                                                             const float* __restrict__ sink, int H, int rank, int n_chunks) {
    const int b = blockIdx.x / H, h = blockIdx.x % H;
    const float* ml = part_ml + (size_t)blockIdx.x * n_chunks * 2;
    float M = sink ? sink[h] * LOG2E : -INFINITY;
    for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, ml[2 * c]);
    float l = sink ? exp2f(sink[h] * LOG2E - M) : 0.0f;
    for (int c = 0; c < n_chunks; ++c)
        if (ml[2 * c + 1] > 0.0f) l += ml[2 * c + 1] * exp2f(ml[2 * c] - M);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    const float* po = part_o + (size_t)blockIdx.x * n_chunks * rank;
    __nv_bfloat16* dst = out + ((size_t)seq_start[b] * H + h) * rank;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        float acc = 0.0f;
        for (int c = 0; c < n_chunks; ++c)
            if (ml[2 * c + 1] > 0.0f) acc = fmaf(po[(size_t)c * rank + i], exp2f(ml[2 * c] - M), acc);
        dst[i] = __float2bfloat16_rn(acc * inv);
    }
}

// How a decode step's keys are shared out: enough blocks for the SMs, at least four tiles (128 keys) each.
void latent_flash_plan(int n_seqs, int H, int window, int max_len, int* chunk_tiles, int* n_chunks) {
    const int span = window > 0 && window < max_len ? window : max_len;
    const int tiles = (span + LF_KEYS - 1) / LF_KEYS + 1;                   // a window may straddle one more tile
    const int blocks = n_seqs * ((H + LF_ROWS - 1) / LF_ROWS);
    int want = (2 * 148 + blocks - 1) / blocks;
    if (want > tiles / 4) want = tiles / 4;
    if (want < 1) want = 1;
    *chunk_tiles = (tiles + want - 1) / want;
    *n_chunks = (tiles + *chunk_tiles - 1) / *chunk_tiles;
}

template <int RANK>
int launch_latent_flash(dim3 grid, cudaStream_t stream, const LfArgs& a) {
    static SpPerDevice ok;
    if (!ok.done()) {
        cudaError_t e = cudaFuncSetAttribute(latent_flash_kernel<RANK>, cudaFuncAttributeMaxDynamicSharedMemorySize, LfSmem<RANK>::TOTAL);
        if (e != cudaSuccess) SP_FAIL("latent_flash: cannot reserve %d bytes of shared memory: %s", LfSmem<RANK>::TOTAL, cudaGetErrorString(e));
        ok.mark();
    }
    latent_flash_kernel<RANK><<<grid, 256, LfSmem<RANK>::TOTAL, stream>>>(a);
    return 0;
}
}  // namespace

SP_API int sp_latent_flash_rows() { return LF_ROWS; }

SP_API int sp_latent_flash_supported(int rank, int page_size) {
    return page_size == LF_PAGE && (rank == 128 || rank == 256 || rank == 384 || rank == 512);
}

// ``decode``: every sequence brings one token (grid: groups of LF_ROWS heads x sequences); else ``n_q_tiles`` = the sum
// over sequences of ceil(new tokens / LF_ROWS).
// Floats of scratch that a decode step of ``n_seqs`` sequences no longer than ``max_len`` needs (0: its keys are not split).
SP_API long long sp_latent_flash_scratch_floats(int n_seqs, int H, int rank, int window, int max_len) {
    int ct, nc;
    latent_flash_plan(n_seqs, H, window, max_len, &ct, &nc);
    return nc > 1 ? (long long)n_seqs * H * nc * (rank + 2) : 0;
}

SP_API int sp_latent_flash(const void* q, void* out, const void* pool, const int* seq_start, const int* positions,
                           const int* seq_row, const int* page_table, int max_pages, int page_size, int n_seqs,
                           int n_q_tiles, int decode, int H, int rank, int window, float scale, const float* sink,
                           int max_len, float* scratch, long long scratch_floats, cudaStream_t stream) {
    if (n_seqs <= 0 || (!decode && n_q_tiles <= 0)) return 0;
    if (!sp_latent_flash_supported(rank, page_size)) SP_FAIL("latent_flash: built for ranks 128, 256, 384, 512 and pages of %d (got %d, %d)", LF_PAGE, rank, page_size);
    if ((((uintptr_t)q) | ((uintptr_t)out) | ((uintptr_t)pool)) & 15) SP_FAIL("latent_flash: operands must start on a 16-byte boundary");
    int chunk_tiles = 0, n_chunks = 1;
    if (decode && scratch && max_len > 0) {
        latent_flash_plan(n_seqs, H, window, max_len, &chunk_tiles, &n_chunks);
        if (n_chunks > 1 && scratch_floats < (long long)n_seqs * H * n_chunks * (rank + 2))
            SP_FAIL("latent_flash: %lld floats of scratch are too few for %d shares of the keys", scratch_floats, n_chunks);
    }
    const dim3 grid = decode ? dim3((H + LF_ROWS - 1) / LF_ROWS, n_seqs, n_chunks) : dim3(H, n_q_tiles);
    if (grid.y > 65535) SP_FAIL("latent_flash: %u rows of blocks are beyond this kernel's grid", grid.y);
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n_seqs * H * n_chunks * rank : nullptr;
    LfArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)pool, page_table, seq_row, max_pages,
             seq_start, positions, n_seqs, sink, H, window, scale * LOG2E, decode ? 1 : 0, sp_range_host,
             n_chunks, chunk_tiles, part_o, part_ml};
    int rc = 1;
    switch (rank) {
        case 128: rc = launch_latent_flash<128>(grid, stream, a); break;
        case 256: rc = launch_latent_flash<256>(grid, stream, a); break;
        case 384: rc = launch_latent_flash<384>(grid, stream, a); break;
        case 512: rc = launch_latent_flash<512>(grid, stream, a); break;
    }
    if (rc) return 1;
    SP_CHECK_LAUNCH("latent_flash");
    if (n_chunks > 1) {
        latent_combine_kernel<<<n_seqs * H, 128, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, seq_start, sink, H, rank, n_chunks);
        SP_CHECK_LAUNCH("latent_combine");
    }
    return 0;
}
