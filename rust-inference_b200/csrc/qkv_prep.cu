// What lies between the q/k/v product and the attention kernels, for attention parts whose projections have biases,
// whose queries and keys are normed AFTER the rotation, or whose values are the keys: one pass over the product.
//
//   proj [tokens, ld]: the product's rows; q heads start at column q_col, k heads at k_col, v heads at v_col
//                      (v_col < 0: there are none; the values are the keys as cached and nothing is written for them),
//                      every head Dp columns wide (Dk true elements, zeros after them)
//   bias [..]:         float32, indexed by the product's column (null: none); added first
//   q_out [tokens, H, Dp];  k_pool, v_pool [pages, KV, page_size, Dp]
//
// For a q or k head x (after the bias), with `norm` 1: x <- x / sqrt(sum(x^2) / Dk + norm_eps) * gain (q_gain, k_gain:
// float32 [Dp], the same for every head); with `norm` 2 the sum runs over ALL q heads (all k heads) of the token at once,
//     x <- x / sqrt(sum over the heads of sum(x^2) / (H Dk) + norm_eps) * gain[h],   gains [H, Dp] and [KV, Dp],
// both before the rotation.  Then the first `rot` elements are turned by the angles of the token's position,
// (c, s) = table[pos][i]: partners are neighbours (2i, 2i+1) with `pairs`, else i and i + rot/2:
//     a' = a c - b s,  b' = b c + a s;
// then, with `unit`, the head is divided by its root mean square over its Dk true elements:
//     x' / sqrt(sum(x'^2) / Dk + eps)                    (no gain);
// q goes to q_out, k to the token's place in its page.  v heads get their bias and are stored.  All of it float32.
#include "common.cuh"

#define QP_WARPS 4
#define QP_MAX_DP 512

struct QpArgs {
    const void* proj;
    long long ld;
    int q_col, k_col, v_col;
    const float* bias;
    void *q_out, *k_pool, *v_pool;
    const int *page_table, *tok_seq, *tok_pos, *seq_slot;
    const float2* rope;
    int rope_rows, rot, pairs, unit;
    float eps;
    const float *q_gain, *k_gain;
    int norm;
    float norm_eps;
    int H, KV, Dp, Dk, mpps, page_size, num_pages, write_kv;
    int* err;
};

// where a token's keys and values go: the page, or -1 (unmapped: reported, the write is skipped)
__device__ __forceinline__ int qp_page(const QpArgs& a, int t, int pos) {
    if (!a.write_kv) return -1;
    const int slot = a.seq_slot[a.tok_seq[t]];
    const int page = a.page_table[(size_t)slot * a.mpps + pos / a.page_size];
    if (page < 0 || page >= a.num_pages) {
        if ((threadIdx.x & 31) == 0) atomicExch(a.err, 2);
        return -1;
    }
    return page;
}

// norm 2: 1 / sqrt(mean of the squares over all q heads' (k heads') true elements + eps), by the whole block, in a
// fixed order; padding columns hold zeros (a zero row of the matrix and a zero of the bias) and add nothing
template <typename T>
__device__ __forceinline__ void qp_whole_norms(const QpArgs& a, const T* row, float* red, float& inv_q, float& inv_k) {
    float sq = 0.0f, sk = 0.0f;
    for (int c = threadIdx.x; c < a.H * a.Dp; c += blockDim.x) {
        const float v = ld_f(row + a.q_col + c) + (a.bias ? a.bias[a.q_col + c] : 0.0f);
        sq += v * v;
    }
    for (int c = threadIdx.x; c < a.KV * a.Dp; c += blockDim.x) {
        const float v = ld_f(row + a.k_col + c) + (a.bias ? a.bias[a.k_col + c] : 0.0f);
        sk += v * v;
    }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    inv_q = a.H ? 1.0f / sqrtf(sq / (float)(a.H * a.Dk) + a.norm_eps) : 1.0f;
    inv_k = a.KV ? 1.0f / sqrtf(sk / (float)(a.KV * a.Dk) + a.norm_eps) : 1.0f;
}

// the same with eight elements per load, for rows of whole 16-byte pieces (every thread's partial sums are added in a
// fixed order: by thread, then over the block)
template <typename T> struct Qp8;
template <typename T>
__device__ __forceinline__ void qp_whole_norms8(const QpArgs& a, const T* row, float* red, float& inv_q, float& inv_k);

// any sizes: a warp per head, lanes strided over the head, the head staged in shared memory
template <typename T>
__global__ void qkv_prep_kernel(QpArgs a) {
    __shared__ float buf[QP_WARPS][QP_MAX_DP];
    __shared__ float red[33];
    pdl_trigger();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = a.tok_pos[t];
    const int page = qp_page(a, t, pos);
    const bool rope_ok = !a.rope || (pos >= 0 && pos < a.rope_rows);
    pdl_wait();
    if (!rope_ok) {
        if (threadIdx.x == 0) atomicExch(a.err, 3);
        return;
    }
    const int Dp = a.Dp, H = a.H, KV = a.KV;
    const int heads_total = H + KV + (a.v_col >= 0 ? KV : 0);
    const int half = a.rot / 2;
    const T* row = (const T*)a.proj + (size_t)t * a.ld;
    float* x = buf[warp];
    float inv_q = 1.0f, inv_k = 1.0f;
    if (a.norm == 2) qp_whole_norms<T>(a, row, red, inv_q, inv_k);
    for (int h = blockIdx.y * QP_WARPS + warp; h < heads_total; h += QP_WARPS * gridDim.y) {
        const int which = h < H ? 0 : (h < H + KV ? 1 : 2);
        const int hh = which == 0 ? h : (which == 1 ? h - H : h - H - KV);
        const int col = (which == 0 ? a.q_col : (which == 1 ? a.k_col : a.v_col)) + hh * Dp;
        T* dst;
        if (which == 0) {
            dst = (T*)a.q_out + ((size_t)t * H + h) * Dp;
        } else {
            if (page < 0) continue;
            dst = (T*)(which == 1 ? a.k_pool : a.v_pool) + (((size_t)page * KV + hh) * a.page_size + pos % a.page_size) * Dp;
        }
        for (int d = lane; d < Dp; d += 32) x[d] = ld_f(row + col + d) + (a.bias ? a.bias[col + d] : 0.0f);
        __syncwarp();
        if (which == 2) {
            for (int d = lane; d < Dp; d += 32) st_f(dst + d, x[d]);
            __syncwarp();
            continue;
        }
        if (a.norm) {
            const float* gain = which == 0 ? a.q_gain : a.k_gain;
            float ninv = which == 0 ? inv_q : inv_k;
            if (a.norm == 1) {
                float ss = 0.0f;
                for (int d = lane; d < Dp; d += 32) ss += x[d] * x[d];
                ninv = 1.0f / sqrtf(warp_sum(ss) / (float)a.Dk + a.norm_eps);
            } else {
                gain += (size_t)hh * Dp;
            }
            for (int d = lane; d < Dp; d += 32) x[d] = x[d] * ninv * gain[d];
            __syncwarp();
        }
        if (a.rope) {
            const float2* cs = a.rope + (size_t)pos * half;
            for (int i = lane; i < half; i += 32) {
                const int ia = a.pairs ? 2 * i : i, ib = a.pairs ? 2 * i + 1 : i + half;
                const float u = x[ia], v = x[ib];
                const float2 c = cs[i];
                x[ia] = u * c.x - v * c.y;
                x[ib] = v * c.x + u * c.y;
            }
            __syncwarp();
        }
        float inv = 1.0f;
        if (a.unit) {
            float ss = 0.0f;
            for (int d = lane; d < Dp; d += 32) ss += x[d] * x[d];
            inv = 1.0f / sqrtf(warp_sum(ss) / (float)a.Dk + a.eps);
        }
        for (int d = lane; d < Dp; d += 32) st_f(dst + d, x[d] * inv);
        __syncwarp();
    }
}

// Heads of whole 8-element pieces with neighbouring rotation partners: a lane holds eight consecutive elements
// (one 16-byte load in bfloat16, two in float32), so a pair's partner is in the same lane.  A head takes Dp / 8 lanes;
// a warp works on 32 / GROUP heads at a time, GROUP = Dp / 8 rounded up to a power of two (lanes past a head's end
// idle), and a head's sum of squares is a butterfly inside its group of lanes.
template <typename T> struct Qp8;
template <> struct Qp8<float> {
    static __device__ __forceinline__ void load(const float* p, float* x) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* x) {
        *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(x[4], x[5], x[6], x[7]);
    }
};
template <> struct Qp8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* x) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __bfloat1622float2(p2[j]);
            x[2 * j] = f.x;
            x[2 * j + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* x) {
        uint4 o;
        unsigned* ow = reinterpret_cast<unsigned*>(&o);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const __nv_bfloat162 pk = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
            ow[j] = *reinterpret_cast<const unsigned*>(&pk);
        }
        *reinterpret_cast<uint4*>(p) = o;
    }
};

template <typename T>
__device__ __forceinline__ void qp_whole_norms8(const QpArgs& a, const T* row, float* red, float& inv_q, float& inv_k) {
    float sq = 0.0f, sk = 0.0f;
    for (int which = 0; which < 2; which++) {
        const int col0 = which ? a.k_col : a.q_col, n8 = (which ? a.KV : a.H) * a.Dp / 8;
        float acc = 0.0f;
        for (int i = threadIdx.x; i < n8; i += blockDim.x) {
            float x[8];
            Qp8<T>::load(row + col0 + 8 * i, x);
            if (a.bias) {
                float b[8];
                Qp8<float>::load(a.bias + col0 + 8 * i, b);
#pragma unroll
                for (int j = 0; j < 8; j++) x[j] += b[j];
            }
#pragma unroll
            for (int j = 0; j < 8; j++) acc += x[j] * x[j];
        }
        if (which) sk = acc; else sq = acc;
    }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    inv_q = a.H ? 1.0f / sqrtf(sq / (float)(a.H * a.Dk) + a.norm_eps) : 1.0f;
    inv_k = a.KV ? 1.0f / sqrtf(sk / (float)(a.KV * a.Dk) + a.norm_eps) : 1.0f;
}

// Partners half a rotated part apart (`pairs` 0) live in another lane of the head's group, rot / 16 lanes away (rot is
// then a multiple of 16, so that a lane's eight elements lie on one side); a lane fetches them by shuffles.
// PAIRS (partners are neighbours, or nothing is turned at all) and NORM (the norm before the rotation: 0, 1, 2) are
// template parameters, so that a variant holds only its own angles and gains in registers.
template <typename T, bool PAIRS, int NORM>
__global__ void qkv_prep_vec_kernel(QpArgs a, int group) {
    __shared__ float red[33];
    pdl_trigger();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hpw = 32 / group;                               // heads a warp works on at a time
    const int sub = lane / group, ln = lane % group;
    const int Dp = a.Dp, H = a.H, KV = a.KV;
    const int d0 = ln * 8;
    const bool live_lane = d0 < Dp;
    const int pos = a.tok_pos[t];
    const int page = qp_page(a, t, pos);
    const bool rope_ok = !a.rope || (pos >= 0 && pos < a.rope_rows);
    // the angles of this lane's four pairs and its share of the bias do not depend on the kernel in front
    float cs_c[4], cs_s[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        cs_c[j] = 1.0f;
        cs_s[j] = 0.0f;
        if (PAIRS && a.rope && rope_ok && live_lane && d0 + 2 * j < a.rot) {
            const float2 c = a.rope[(size_t)pos * (a.rot / 2) + d0 / 2 + j];
            cs_c[j] = c.x;
            cs_s[j] = c.y;
        }
    }
    // halves: this lane's eight angles, the side it is on (the sine's sign) and how far away its partners are
    const int half = a.rot / 2;
    const bool turns = !PAIRS && a.rope && live_lane && d0 < a.rot;
    const bool upper = d0 >= half;
    float hc[8], hs[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        hc[j] = 1.0f;
        hs[j] = 0.0f;
        if (turns && rope_ok) {
            const float2 c = a.rope[(size_t)pos * half + (upper ? d0 - half : d0) + j];
            hc[j] = c.x;
            hs[j] = upper ? c.y : -c.y;
        }
    }
    const int partner = turns ? (upper ? lane - half / 8 : lane + half / 8) : lane;
    float gq[8], gk[8];
#pragma unroll
    for (int j = 0; j < 8; j++) gq[j] = gk[j] = 1.0f;
    if (NORM == 1 && live_lane) {
        if (a.q_gain) Qp8<float>::load(a.q_gain + d0, gq);
        if (a.k_gain) Qp8<float>::load(a.k_gain + d0, gk);
    }
    pdl_wait();
    if (!rope_ok) {
        if (threadIdx.x == 0) atomicExch(a.err, 3);
        return;
    }
    const int heads_total = H + KV + (a.v_col >= 0 ? KV : 0);
    const T* row = (const T*)a.proj + (size_t)t * a.ld;
    float inv_q = 1.0f, inv_k = 1.0f;
    if (NORM == 2) qp_whole_norms8<T>(a, row, red, inv_q, inv_k);
    const int stride = QP_WARPS * hpw * gridDim.y;
    for (int h0 = (blockIdx.y * QP_WARPS + warp) * hpw; h0 < heads_total; h0 += stride) {
        const int h = h0 + sub;
        // (no lane leaves early: the shuffles below are the whole warp's)
        const bool live = live_lane && sub < hpw && h < heads_total;
        const int which = !live ? 3 : (h < H ? 0 : (h < H + KV ? 1 : 2));
        const int hh = which == 0 ? h : (which == 1 ? h - H : h - H - KV);
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; j++) x[j] = 0.0f;
        T* dst = nullptr;
        if (live) {
            const int col = (which == 0 ? a.q_col : (which == 1 ? a.k_col : a.v_col)) + hh * Dp + d0;
            Qp8<T>::load(row + col, x);
            if (a.bias) {
                const float4 b0 = *reinterpret_cast<const float4*>(a.bias + col), b1 = *reinterpret_cast<const float4*>(a.bias + col + 4);
                x[0] += b0.x; x[1] += b0.y; x[2] += b0.z; x[3] += b0.w; x[4] += b1.x; x[5] += b1.y; x[6] += b1.z; x[7] += b1.w;
            }
            if (which == 0) dst = (T*)a.q_out + ((size_t)t * H + h) * Dp + d0;
            else if (page >= 0)
                dst = (T*)(which == 1 ? a.k_pool : a.v_pool) + (((size_t)page * KV + hh) * a.page_size + pos % a.page_size) * Dp + d0;
        }
        if (NORM) {
            float ninv = which == 0 ? inv_q : inv_k;
            if (NORM == 1) {
                float ss = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; j++) ss += x[j] * x[j];
                for (int o = group >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                ninv = 1.0f / sqrtf(ss / (float)a.Dk + a.norm_eps);
            }
            if (which < 2) {
                float g8[8];
                if (NORM == 2) {
                    Qp8<float>::load((which == 0 ? a.q_gain : a.k_gain) + (size_t)hh * Dp + d0, g8);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j++) g8[j] = which == 0 ? gq[j] : gk[j];
                }
#pragma unroll
                for (int j = 0; j < 8; j++) x[j] = x[j] * ninv * g8[j];
            }
        }
        if (!PAIRS) {
            // every lane takes part in the shuffles; a lane that does not turn keeps its own values (cos 1, sin 0)
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float other = __shfl_sync(0xffffffffu, x[j], partner);
                if (which < 2) x[j] = x[j] * hc[j] + other * hs[j];
            }
        } else if (which < 2) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float u = x[2 * j], v = x[2 * j + 1];
                x[2 * j] = u * cs_c[j] - v * cs_s[j];
                x[2 * j + 1] = v * cs_c[j] + u * cs_s[j];
            }
        }
        if (a.unit) {
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) ss += x[j] * x[j];
            for (int o = group >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (which < 2) {
                const float inv = 1.0f / sqrtf(ss / (float)a.Dk + a.eps);
#pragma unroll
                for (int j = 0; j < 8; j++) x[j] *= inv;
            }
        }
        if (dst) Qp8<T>::store(dst, x);
    }
}

extern "C" int ri_qkv_prep(const void* proj, long long ld, int q_col, int k_col, int v_col, const float* bias, void* q_out,
                           void* k_pool, void* v_pool, const int* page_table, const int* tok_seq, const int* tok_pos,
                           const int* seq_slot, const float* rope_table, int rope_rows, int rot, int pairs, int unit,
                           float eps, int tokens, int H, int KV, int Dp, int Dk, int mpps, int page_size, int num_pages,
                           int write_kv, int dtype, int* err_flag, cudaStream_t stream);

// The same with a norm of q and k heads before the rotation: norm 1 per head (gains [Dp]), 2 over all heads of the
// token at once (gains [H, Dp] and [KV, Dp]); 0: none.
extern "C" int ri_qkv_prep_norm(const void* proj, long long ld, int q_col, int k_col, int v_col, const float* bias, void* q_out,
                                void* k_pool, void* v_pool, const int* page_table, const int* tok_seq, const int* tok_pos,
                                const int* seq_slot, const float* rope_table, int rope_rows, int rot, int pairs, int unit,
                                float eps, const float* q_gain, const float* k_gain, int norm, float norm_eps, int tokens,
                                int H, int KV, int Dp, int Dk, int mpps, int page_size, int num_pages, int write_kv,
                                int dtype, int* err_flag, cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(norm >= 0 && norm <= 2, "qkv_prep: norm %d", norm);
    RI_REQUIRE(!norm || ((q_gain || !H) && (k_gain || !KV)), "qkv_prep: a norm needs its gains");
    RI_REQUIRE(tokens > 0 && H >= 0 && KV >= 0 && H + KV > 0 && Dp > 0 && Dk > 0 && Dk <= Dp, "qkv_prep: bad sizes");
    RI_REQUIRE(Dp <= QP_MAX_DP, "qkv_prep: heads of %d elements exceed the limit %d", Dp, QP_MAX_DP);
    RI_REQUIRE(rot >= 0 && rot <= Dk && rot % 2 == 0, "qkv_prep: %d rotated elements must be even and within the head's %d", rot, Dk);
    RI_REQUIRE(!rope_table || rot > 0, "qkv_prep: a rotation table needs rotated elements");
    RI_REQUIRE(page_size > 0 && mpps > 0, "qkv_prep: bad page sizes");
    RI_REQUIRE(dtype == RI_DTYPE_F32 || dtype == RI_DTYPE_BF16, "qkv_prep: unknown dtype %d", dtype);
    if (KV == 0) write_kv = 0;
    QpArgs a;
    a.proj = proj; a.ld = ld; a.q_col = q_col; a.k_col = k_col; a.v_col = v_col; a.bias = bias; a.q_out = q_out;
    a.k_pool = k_pool; a.v_pool = v_pool; a.page_table = page_table; a.tok_seq = tok_seq; a.tok_pos = tok_pos;
    a.seq_slot = seq_slot; a.rope = (const float2*)rope_table; a.rope_rows = rope_rows; a.rot = rope_table ? rot : 0;
    a.q_gain = q_gain; a.k_gain = k_gain; a.norm = norm; a.norm_eps = norm_eps;
    a.pairs = pairs; a.unit = unit; a.eps = eps; a.H = H; a.KV = KV; a.Dp = Dp; a.Dk = Dk; a.mpps = mpps;
    a.page_size = page_size; a.num_pages = num_pages; a.write_kv = write_kv; a.err = err_flag;
    const int heads_total = H + KV + (v_col >= 0 ? KV : 0);
    const int es = dtype == RI_DTYPE_F32 ? 4 : 2;
    // every piece of eight elements must start on 16 bytes: the row pitch, the columns, the heads and the pointers
    const bool vec = Dp % 8 == 0 && Dp <= 256 && (pairs || !rope_table || rot % 16 == 0) && (ld * es) % 16 == 0 &&
                     (q_col * es) % 16 == 0 && (k_col * es) % 16 == 0 && (v_col < 0 || (v_col * es) % 16 == 0) &&
                     ((((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)bias |
                        (uintptr_t)q_gain | (uintptr_t)k_gain) & 15) == 0);
    if (vec) {
        int group = 1;
        while (group < Dp / 8) group <<= 1;
        const int per_block = QP_WARPS * (32 / group);
        int hb = (heads_total + per_block - 1) / per_block;
        if ((long long)tokens * hb > 4096) hb = 1 > 4096 / tokens ? 1 : 4096 / tokens;
        // (norm 2: every block of a token adds up the token's whole q and k projections for itself, in the same order,
        // so the blocks of a token agree bit for bit; the rows come from L2)
        RI_REQUIRE(hb <= 65535, "qkv_prep: bad grid");
        dim3 grid(tokens, hb);
        const bool as_pairs = pairs || !rope_table;          // nothing to turn: the variant without shuffles
#define QP_VEC(T, P, N) ri_launch_pdl(qkv_prep_vec_kernel<T, P, N>, grid, dim3(32 * QP_WARPS), 0, stream, a, group)
#define QP_VEC_BY_NORM(T, P)                                 \
        do {                                                 \
            if (norm == 0) QP_VEC(T, P, 0);                  \
            else if (norm == 1) QP_VEC(T, P, 1);             \
            else QP_VEC(T, P, 2);                            \
        } while (0)
        if (dtype == RI_DTYPE_F32) {
            if (as_pairs) QP_VEC_BY_NORM(float, true); else QP_VEC_BY_NORM(float, false);
        } else {
            if (as_pairs) QP_VEC_BY_NORM(__nv_bfloat16, true); else QP_VEC_BY_NORM(__nv_bfloat16, false);
        }
#undef QP_VEC_BY_NORM
#undef QP_VEC
        RI_CHECK_LAUNCH("qkv_prep");
        return 0;
    }
    int hb = (heads_total + QP_WARPS - 1) / QP_WARPS;
    if ((long long)tokens * hb > 4096) hb = 1 > 4096 / tokens ? 1 : 4096 / tokens;
    RI_REQUIRE(hb <= 65535, "qkv_prep: bad grid");
    dim3 grid(tokens, hb);
    if (dtype == RI_DTYPE_F32) ri_launch_pdl(qkv_prep_kernel<float>, grid, dim3(32 * QP_WARPS), 0, stream, a);
    else ri_launch_pdl(qkv_prep_kernel<__nv_bfloat16>, grid, dim3(32 * QP_WARPS), 0, stream, a);
    RI_CHECK_LAUNCH("qkv_prep");
    return 0;
}

extern "C" int ri_qkv_prep(const void* proj, long long ld, int q_col, int k_col, int v_col, const float* bias, void* q_out,
                           void* k_pool, void* v_pool, const int* page_table, const int* tok_seq, const int* tok_pos,
                           const int* seq_slot, const float* rope_table, int rope_rows, int rot, int pairs, int unit,
                           float eps, int tokens, int H, int KV, int Dp, int Dk, int mpps, int page_size, int num_pages,
                           int write_kv, int dtype, int* err_flag, cudaStream_t stream) {
    return ri_qkv_prep_norm(proj, ld, q_col, k_col, v_col, bias, q_out, k_pool, v_pool, page_table, tok_seq, tok_pos, seq_slot,
                            rope_table, rope_rows, rot, pairs, unit, eps, nullptr, nullptr, 0, 0.0f, tokens, H, KV, Dp, Dk,
                            mpps, page_size, num_pages, write_kv, dtype, err_flag, stream);
}
