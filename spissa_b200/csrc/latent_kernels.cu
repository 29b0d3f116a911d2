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
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x)
        sp_st_dt(a.pool, a.pool_dt, base + i, lat[i] * inv_c * sp_ld_dt(a.wc, a.w_dt, i));
}

SP_API int sp_latent_norm_store(const float* proj, int ld, const void* wq, const void* wc, int w_dt, void* cq, int cq_dt,
                                void* pool, int pool_dt, const int* token_seq, const int* positions, const int* seq_row,
                                const int* page_table, int max_pages, int page_size, int T, int qr, int rank, float eps,
                                cudaStream_t stream) {
    if (T <= 0) return 0;
    if (qr <= 0 || rank <= 0 || ld < qr + (pool ? rank : 0)) SP_FAIL("latent_norm_store: parts of %d and %d do not fit rows of %d", qr, rank, ld);
    LnArgs a{proj, ld, wq, wc, w_dt, cq, cq_dt, pool, pool_dt, token_seq, positions, seq_row, page_table, max_pages,
             page_size, T, qr, rank, eps, sp_range_host};
    latent_norm_store_kernel<<<T, 256, 0, stream>>>(a);
    SP_CHECK_LAUNCH("latent_norm_store");
    return 0;
}

// ============================================================== a stack of small matrices, one per head
// out[t][h][n] = Σ_k a[t][h][k] · W_h[k][n]. ``w`` holds the heads' matrices one after another, either as rows of k
// (w[h][k][n], ``w_rows_are_k``) or as rows of n (w[h][n][k]): a slice [h·N … (h+1)·N) of rows of a matrix stored
// [out, in]. A block takes HW_TT tokens x HW_TN outputs of one head; a and W pass through shared memory in blocks
// of HW_TK of k; a thread owns one output column for all the block's tokens and adds over k in ascending order.
#define HW_TT 32
#define HW_TN 128
#define HW_TK 32
template <typename TA, typename TW, typename TO>
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
            for (int e = tid; e < HW_TK * HW_TN; e += HW_TN) {
                const int kk = e / HW_TN, nn = e % HW_TN;
                const int k = k0 + kk, n = n0 + nn;
                Ws[kk][nn] = (k < K && n < N) ? sp_ld(wh, (size_t)k * N + n) : 0.0f;
            }
        } else {
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

SP_API int sp_headwise_product(const void* a, int a_dt, const void* w, int w_dt, void* out, int out_dt, int T, int H, int K,
                               int N, int w_rows_are_k, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || K <= 0 || N <= 0) SP_FAIL("headwise_product: sizes %d x %d x %d", H, K, N);
    const dim3 grid((T + HW_TT - 1) / HW_TT, H, (N + HW_TN - 1) / HW_TN);
    if (grid.y > 65535 || grid.z > 65535) SP_FAIL("headwise_product: %d heads or %d outputs are too many for one launch", H, N);
#define HW_LAUNCH(TA, TW, TO) headwise_product_kernel<TA, TW, TO><<<grid, HW_TN, 0, stream>>>((const TA*)a, (const TW*)w, (TO*)out, T, H, K, N, w_rows_are_k)
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
