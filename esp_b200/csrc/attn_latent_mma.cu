// Attention over cached latent rows on the tensor cores (bfloat16 in, float out): the many-row and few-row
// form of attn_latent in latent.cu for bfloat16 engines.  All query heads read the same cached rows (keys: the whole
// row of hdk channels; values: its first hdv channels), so the rows of a tile are (token, head) pairs: a block
// owns 32 of them (32 / HG consecutive new tokens of one sequence times HG heads), walks the sequence's pages of
// 64 positions in ascending order, and keeps running maximum, sum and weighted values in float registers.
//
// Eight warps: two groups of 16 rows times four quarters.  For a page, warp (group, quarter) takes the scores
// of its 16 rows against 16 of the 64 keys (mma.sync m16n8k16 over hdk), the quarters exchange row maxima and sums
// and the rounded weights through shared memory, and then every warp adds P V for its share of the value channels
// (pairs of 8-channel tiles dealt round robin to the quarters), so a row's 512 value channels cost 64 registers a
// thread.  Pages arrive by cp.async, the next one while the current one is used.  hdk and hdv are multiples of 16,
// hdv at most 512; the page size is 64.
#include "common.cuh"

namespace {
constexpr int ROWS = 32, BN = 64, THREADS = 256;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;          // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// NP: pairs of value tiles (16 channels) a warp may own: hdv <= 64 * NP
template <int NP>
__global__ void __launch_bounds__(THREADS)
attn_latent_mma_kernel(const bf16* __restrict__ qx, const bf16* __restrict__ pool, bf16* __restrict__ out,
                       const int* __restrict__ tile_seq, const int* __restrict__ tile_first,
                       const int* __restrict__ seq_start, const int* __restrict__ seq_past,
                       const int* __restrict__ block_table, int table_stride, int n_pages, int H, int hg, int hdk, int hdv,
                       int window, float scale, int n_splits, int pages_per_split, float* __restrict__ part_o,
                       float* __restrict__ part_ml, int* __restrict__ status) {
    pdl_trigger();
    const int lds = hdk + 8;                         // row stride in elements: 16 bytes of padding against bank conflicts
    constexpr int LDP = BN + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* k_s = reinterpret_cast<bf16*>(smem_raw);                    // [2][BN][lds]
    bf16* q_s = k_s + 2 * BN * lds;                                    // [ROWS][lds]
    bf16* p_s = q_s + ROWS * lds;                                      // [ROWS][LDP]
    float* smax = reinterpret_cast<float*>(p_s + ROWS * LDP);          // [4][ROWS]
    float* ssum = smax + 4 * ROWS;                                     // [4][ROWS]

    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;             // later tiles see more keys: they start first
    const int h0 = blockIdx.y * hg;
    const int tq = ROWS / hg;                                          // new tokens of a tile
    const int seq = tile_seq[tile], first = tile_first[tile];
    const int row0 = seq_start[seq] + first;
    const int n_new = seq_start[seq + 1] - seq_start[seq];
    const int count = min(tq, n_new - first);
    const int pos0 = seq_past[seq] + first, pos_last = pos0 + count - 1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tg = lane & 3;
    const int rg = warp >> 2, qt = warp & 3;
    const int pieces = hdk / 8;

    pdl_wait();
    // ---- the tile's queries -> shared memory (rows beyond the tile's tokens or the heads are zero)
    for (int idx = tid; idx < ROWS * pieces; idx += THREADS) {
        const int r = idx / pieces, p = idx - r * pieces;
        const int t = r / hg, h = h0 + r % hg;
        const bool ok = t < count && h < H;
        cp_async16(q_s + r * lds + p * 8, qx + ((size_t)(row0 + (ok ? t : 0)) * H + (ok ? h : 0)) * hdk + p * 8, ok);
    }
    cp_async_commit();

    const int key_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    int blk_lo = key_lo / BN, blk_hi = pos_last / BN;
    if (n_splits > 1) {                              // this block's share of the tile's pages (it may be empty)
        blk_lo += (int)blockIdx.z * pages_per_split;
        blk_hi = min(blk_hi, blk_lo + pages_per_split - 1);
    }

    auto load_page = [&](int blk, int buf) {
        int pg = block_table[(size_t)seq * table_stride + blk];
        const bool pg_ok = pg >= 0 && pg < n_pages;
        if (!pg_ok) {
            if (tid == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
            pg = 0;
        }
        const bf16* src = pool + (size_t)pg * BN * hdk;
        for (int idx = tid; idx < BN * pieces; idx += THREADS) {
            const int r = idx / pieces, p = idx - r * pieces;
            cp_async16(k_s + (buf * BN + r) * lds + p * 8, src + (size_t)r * hdk + p * 8, pg_ok);
        }
        cp_async_commit();
    };
    if (blk_lo <= blk_hi) load_page(blk_lo, 0);

    float o[2 * NP][4];
#pragma unroll
    for (int i = 0; i < 2 * NP; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) o[i][j] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float log2e = 1.4426950408889634f;
    // this lane's two rows of its group: token, validity, position
    int my_pos[2];
    bool my_ok[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = rg * 16 + g + 8 * r;
        const int t = row / hg, h = h0 + row % hg;
        my_ok[r] = t < count && h < H;
        my_pos[r] = pos0 + t;
    }
    const int n_pairs = hdv / 16;
    const int ksteps = hdk / 16;

    for (int blk = blk_lo; blk <= blk_hi; blk++) {
        const int buf = (blk - blk_lo) & 1;
        __syncthreads();                          // the page before and its weights are no longer read
        if (blk < blk_hi) load_page(blk + 1, buf ^ 1);
        if (blk < blk_hi) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();
        const bf16* kb = k_s + buf * BN * lds;

        // scores of 16 rows against this quarter's 16 keys
        float s[2][4];
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) s[i][j] = 0.f;
        for (int kk = 0; kk < ksteps; kk++) {
            unsigned qf[4], kf[4];
            ldmatrix_x4(qf, q_s + (rg * 16 + (lane & 15)) * lds + kk * 16 + (lane >> 4) * 8);
            ldmatrix_x4(kf, kb + (qt * 16 + (lane & 7) + (lane >> 4) * 8) * lds + kk * 16 + ((lane >> 3) & 1) * 8);
            mma16816(s[0], qf, kf[0], kf[1]);
            mma16816(s[1], qf, kf[2], kf[3]);
        }
        const int key0 = blk * BN + qt * 16;
        float m_part[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int r = j >> 1;
                const int key = key0 + nt * 8 + tg * 2 + (j & 1);
                const bool seen = my_ok[r] && key <= my_pos[r] && (window <= 0 || my_pos[r] - key < window);
                const float v = seen ? s[nt][j] * scale : -INFINITY;
                s[nt][j] = v;
                m_part[r] = fmaxf(m_part[r], v);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; r++) {
            m_part[r] = fmaxf(m_part[r], __shfl_xor_sync(0xffffffffu, m_part[r], 1));
            m_part[r] = fmaxf(m_part[r], __shfl_xor_sync(0xffffffffu, m_part[r], 2));
            if (tg == 0) smax[qt * ROWS + rg * 16 + g + 8 * r] = m_part[r];
        }
        __syncthreads();
        float scale_old[2], m_use[2], l_part[2] = {0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int row = rg * 16 + g + 8 * r;
            float m_new = fmaxf(fmaxf(smax[row], smax[ROWS + row]), fmaxf(smax[2 * ROWS + row], smax[3 * ROWS + row]));
            m_new = fmaxf(m_new, m_run[r]);
            m_use[r] = m_new == -INFINITY ? 0.f : m_new;
            scale_old[r] = exp2f((m_run[r] - m_use[r]) * log2e);       // m_run = -inf gives 0
            m_run[r] = m_new;
        }
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            float p[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                p[j] = exp2f((s[nt][j] - m_use[j >> 1]) * log2e);
                l_part[j >> 1] += p[j];
            }
            bf16* dst = p_s + (rg * 16 + g) * LDP + qt * 16 + nt * 8 + tg * 2;
            *reinterpret_cast<unsigned*>(dst) = pack_bf16(p[0], p[1]);
            *reinterpret_cast<unsigned*>(dst + 8 * LDP) = pack_bf16(p[2], p[3]);
        }
#pragma unroll
        for (int r = 0; r < 2; r++) {
            l_part[r] += __shfl_xor_sync(0xffffffffu, l_part[r], 1);
            l_part[r] += __shfl_xor_sync(0xffffffffu, l_part[r], 2);
            if (tg == 0) ssum[qt * ROWS + rg * 16 + g + 8 * r] = l_part[r];
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int row = rg * 16 + g + 8 * r;
            l_run[r] = l_run[r] * scale_old[r] + ((ssum[row] + ssum[ROWS + row]) + (ssum[2 * ROWS + row] + ssum[3 * ROWS + row]));
        }
#pragma unroll
        for (int i = 0; i < 2 * NP; i++) {
            o[i][0] *= scale_old[0];
            o[i][1] *= scale_old[0];
            o[i][2] *= scale_old[1];
            o[i][3] *= scale_old[1];
        }
        // O += P V for this quarter's channel pairs
#pragma unroll
        for (int kt = 0; kt < BN / 16; kt++) {
            unsigned pf[4];
            ldmatrix_x4(pf, p_s + (rg * 16 + (lane & 15)) * LDP + kt * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int i = 0; i < NP; i++) {
                const int pair = qt + 4 * i;
                if (pair < n_pairs) {
                    unsigned vf[4];
                    ldmatrix_x4_trans(vf, kb + (kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * lds + pair * 16 + (lane >> 4) * 8);
                    mma16816(o[2 * i], pf, vf[0], vf[1]);
                    mma16816(o[2 * i + 1], pf, vf[2], vf[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    // ---- a share of the keys: maximum, sum and unnormalised values go to scratch; the combine kernel finishes
    if (n_splits > 1) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
            if (!my_ok[r]) continue;
            const int row = rg * 16 + g + 8 * r;
            const int t = row / hg, h = h0 + row % hg;
            const size_t slot = ((size_t)(row0 + t) * H + h) * n_splits + blockIdx.z;
            if (qt == 0 && tg == 0) {
                part_ml[2 * slot] = m_run[r];
                part_ml[2 * slot + 1] = l_run[r];
            }
            float* dst = part_o + slot * hdv;
#pragma unroll
            for (int i = 0; i < NP; i++) {
                const int pair = qt + 4 * i;
                if (pair < n_pairs) {
#pragma unroll
                    for (int half = 0; half < 2; half++)
                        *reinterpret_cast<float2*>(dst + pair * 16 + half * 8 + tg * 2) =
                            make_float2(o[2 * i + half][2 * r], o[2 * i + half][2 * r + 1]);
                }
            }
        }
        return;
    }
    // ---- write the rows out
#pragma unroll
    for (int r = 0; r < 2; r++) {
        if (!my_ok[r]) continue;
        const int row = rg * 16 + g + 8 * r;
        const int t = row / hg, h = h0 + row % hg;
        const float inv = l_run[r] > 0.f ? 1.0f / l_run[r] : 0.f;
        bf16* dst = out + ((size_t)(row0 + t) * H + h) * hdv;
#pragma unroll
        for (int i = 0; i < NP; i++) {
            const int pair = qt + 4 * i;
            if (pair < n_pairs) {
#pragma unroll
                for (int half = 0; half < 2; half++)
                    *reinterpret_cast<unsigned*>(dst + pair * 16 + half * 8 + tg * 2) =
                        pack_bf16(o[2 * i + half][2 * r] * inv, o[2 * i + half][2 * r + 1] * inv);
            }
        }
    }
}

// out[n, h] = sum_s w_s O_s / sum_s w_s l_s with w_s = exp(m_s - max m), splits added in ascending order.  A warp a row.
__global__ void __launch_bounds__(128)
attn_latent_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out, int rows,
                           int n_splits, int hdv) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float wts[];                  // [n_splits] weights of the splits, then their sum
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* ml = part_ml + (size_t)row * n_splits * 2;
    if (tid < 32) {
        float m = -INFINITY;
        for (int s = tid; s < n_splits; s += 32) m = fmaxf(m, ml[2 * s]);
        m = warp_max(m);
        for (int s = tid; s < n_splits; s += 32) wts[s] = ml[2 * s] == -INFINITY ? 0.f : expf(ml[2 * s] - m);
        __syncwarp();
        if (tid == 0) {
            float l = 0.f;
            for (int s = 0; s < n_splits; s++) l = fmaf(wts[s], ml[2 * s + 1], l);
            wts[n_splits] = l > 0.f ? 1.0f / l : 0.f;
        }
    }
    __syncthreads();
    const float inv = wts[n_splits];
    const float* po = part_o + (size_t)row * n_splits * hdv;
    for (int c = tid * 4; c < hdv; c += blockDim.x * 4) {     // four channels a thread, every split's piece one 16-byte load
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int s = 0; s < n_splits; s++) {
            const float4 v = *reinterpret_cast<const float4*>(po + (size_t)s * hdv + c);
            const float ws = wts[s];
            acc.x = fmaf(ws, v.x, acc.x);
            acc.y = fmaf(ws, v.y, acc.y);
            acc.z = fmaf(ws, v.z, acc.z);
            acc.w = fmaf(ws, v.w, acc.w);
        }
        bf16* dst = out + (size_t)row * hdv + c;
        *reinterpret_cast<unsigned*>(dst) = pack_bf16(acc.x * inv, acc.y * inv);
        *reinterpret_cast<unsigned*>(dst + 2) = pack_bf16(acc.z * inv, acc.w * inv);
    }
}

template <int NP>
int launch(const void* qx, const void* pool, void* out, const int* tile_seq, const int* tile_first, const int* seq_start,
           const int* seq_past, const int* block_table, int table_stride, int n_pages, int n_tiles, int H, int hg, int hdk,
           int hdv, int window, float scale, int n_splits, int pages_per_split, float* part_o, float* part_ml, int* status,
           cudaStream_t stream) {
    const size_t smem = ((size_t)(2 * BN + ROWS) * (hdk + 8) + (size_t)ROWS * (BN + 8)) * sizeof(bf16) + 8 * ROWS * sizeof(float);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    auto kernel = attn_latent_mma_kernel<NP>;
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); set = true; }
    dim3 grid(n_tiles, (H + hg - 1) / hg, n_splits);
    // many tiles: a long kernel that fills the device, launched the ordinary way; few (decoding): set up under its predecessor
    esp_launch_pdl(n_tiles > 64 ? 0 : ESP_PDL_ATTENTION, kernel, grid, dim3(THREADS), smem, stream, (const bf16*)qx, (const bf16*)pool, (bf16*)out,
                   tile_seq, tile_first, seq_start, seq_past, block_table, table_stride, n_pages, H, hg, hdk, hdv, window, scale,
                   n_splits, pages_per_split, part_o, part_ml, status);
    return esp_launch_status();
}
}  // namespace

// qx [N, H, hdk], pool [pages, 64, hdk], out [N, H, hdv], all bfloat16.  tile_seq / tile_first: tiles of 32 / hg new
// tokens of one sequence (hg: heads of a tile, a power of two up to 32).  n_splits > 1: every tile's pages are dealt to
// n_splits blocks, pages_per_split each, whose partial results (part_o float [N, H, n_splits, hdv], part_ml float
// [N, H, n_splits, 2]) a second kernel combines.
ESP_API int esp_attn_latent_mma(const void* qx, const void* pool, void* out, const int* tile_seq, const int* tile_first,
                                const int* seq_start, const int* seq_past, const int* block_table, int table_stride,
                                int n_pages, int page, int n_tiles, int n_rows, int H, int hg, int hdk, int hdv, int window,
                                float scale, int n_splits, int pages_per_split, float* part_o, float* part_ml, int* status,
                                cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && (!part_o || !part_ml || pages_per_split < 1)))
        return (int)cudaErrorInvalidValue;
    if (page != BN || hdk % 16 || hdv % 16 || hdv > hdk || hdv > 512 || hg <= 0 || hg > ROWS || (hg & (hg - 1)) || H <= 0)
        return (int)cudaErrorInvalidValue;
#define ESP_GO(NP_) code = launch<NP_>(qx, pool, out, tile_seq, tile_first, seq_start, seq_past, block_table, table_stride, \
                                      n_pages, n_tiles, H, hg, hdk, hdv, window, scale, n_splits, pages_per_split, part_o,   \
                                      part_ml, status, stream)
    int code;
    if (hdv <= 64) ESP_GO(1);
    else if (hdv <= 128) ESP_GO(2);
    else if (hdv <= 256) ESP_GO(4);
    else ESP_GO(8);
#undef ESP_GO
    if (code != 0 || n_splits == 1) return code;
    const long long rows = (long long)n_rows * H;
    if ((size_t)(n_splits + 1) * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
    const int threads = hdv / 4 >= 128 ? 128 : (hdv / 4 + 31) / 32 * 32;
    esp_launch_pdl(ESP_PDL_ATTENTION, attn_latent_combine_kernel, dim3((unsigned)rows), dim3(threads),
                   (size_t)(n_splits + 1) * sizeof(float), stream,
                   (const float*)part_o, (const float*)part_ml, (bf16*)out, (int)rows, n_splits, hdv);
    return esp_launch_status();
}
