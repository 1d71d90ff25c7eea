// Gated linear attention: a matrix-valued state per (sequence, head) that every token decays, feeds and reads.
//
//   a_t[d] = sigmoid(z_t[d] + bias[d])^(1/tau)                     decay of key channel d, in (0, 1)
//   S_t[d, j] = a_t[d] S_(t-1)[d, j] + k_t[d] v_t[j]               state [dim, vdim], float32, zero at a sequence's start
//   o_t[j] = sum over d of S_t[d, j] (q_t[d] qscale)               d ascending, one accumulator
// then per head  y_t = o_t / sqrt(mean_j(o_t[j]^2) + eps) * gain * silu(g_t)   (`gla_head_norm_gate`).
//
// `gla_recurrent`: a block owns one (sequence, head, tile of value columns j) and walks the sequence's new
// tokens in order; a thread owns one column of the state (in registers for heads of up to 128 key channels, else in
// shared memory), loaded from / stored to the sequence's slot of the state tensor at the ends.  The decay is computed as
// exp(log_sigmoid(z) / tau) with float32 functions; q, k, v and z come from bfloat16 or float32 projections and
// are widened once.  A token's result depends on the tokens before it only through the state, so prompts,
// pieces of prompts and single tokens give the same bits.
//
// The same kernels run a second form (`gates` given): one decay per token and head instead of one per key channel, and
// a factor on the key,
//   S_t[d, j] = a_t S_(t-1)[d, j] + (b_t k_t[d]) v_t[j],      (a_t, b_t) = gates[t, h, 0..1], float32, made by the caller,
// optionally with one more column j = vdim whose value is 1 for every token (`ones`): that column of the state is the
// running sum n_t = a_t n_(t-1) + b_t k_t, and its output n_t . q_t, which a normaliser behind the kernel reads.  State
// and output are then [.., vdim + 1] wide.
//
//   proj [tokens, ld]: q of head h at columns q_col + h dim .., k at k_col + h dim .., v at v_col + h vdim ..
//   z    [tokens, H dim] (the low-rank decay projection, bias not yet added);  bias [H dim] float32
//   state [slots, H, dim, vdim] float32;  o [tokens, H, vdim] float32
#include "common.cuh"

#define GLA_TILE 64
#define GLA_COLS 256            // threads per block of the register kernel

__device__ __forceinline__ float gla_decay(float z, float inv_tau) {
    // log(sigmoid(z)) = min(z, 0) - log1p(exp(-|z|))
    const float ls = fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
    return expf(ls * inv_tau);
}

// The kernel for heads of up to 128 key channels.  A block of 256 threads owns 16 value columns of the state, and
// sixteen threads share a column: each keeps a sixteenth of the column's key channels in registers (DIMC / 16 of
// them, DIMC the head's key channels rounded up to 64 or 128; channels past `dim` hold zeros and stay zero).  The
// sixteen are four neighbouring lanes in each of four warps (part p = 4 (warp % 4) + lane % 4 has channels
// 64 c + 4 p .. + 3 for c = 0, 1, ..; warps 4 i .. 4 i + 3 own columns 8 i .. 8 i + 7), so that a warp's loads and
// stores of the state cover 8 neighbouring columns, and what the block stages per token serves 16 columns.
// Many small threads instead of few large ones: the recurrence has little to do in parallel (heads x columns), and
// this way a prompt of one sequence still puts some warps on every SM.
// The block stages the decay, key and scaled query of GROUP tokens in shared memory (two buffers): the loads of the
// next group are on their way while the current group is computed, and the decay's exponentials are taken when a
// group is stored.  A group that the sequence does not fill is padded with tokens of decay 1 and key 0, which leave
// the state as it is, bit for bit.  A thread walks its channels in the outer loop and the group's tokens in the
// inner one,
//     S[d] = a_g[d] S[d] + k_g[d] v_g;  acc_g += S[d] q_g[d]            g = 0 .. GROUP-1
// so that neighbouring instructions belong to different accumulators; at the end of the group the partial sums are
// added: the four lanes of a warp by shuffles (pairs first, then the pairs), the four warps through shared memory in
// warp order.  Every token's sum thus has one order that depends on the head's size only: prompts, pieces of
// prompts and single tokens give the same bits (GROUP = 1, for steps in which every sequence brings one token,
// walks the same order).
#define GLA_SPLIT 4             // lanes of a warp that share a column
#define GLA_WARPS 4             // ... and warps
#define GLA_BCOLS (GLA_COLS / GLA_SPLIT / GLA_WARPS)
template <typename T, int DIMC, int GROUP>
__global__ void __launch_bounds__(GLA_COLS)
gla_recurrent_reg_kernel(const T* __restrict__ proj, long long ld, int q_col, int k_col, int v_col,
                         const T* __restrict__ z, const float* __restrict__ bias, float inv_tau, float qscale,
                         float* __restrict__ state, float* __restrict__ o, const int* __restrict__ seq_slot,
                         const int* __restrict__ seq_start, int H, int dim, int vdim_in, const float* __restrict__ gates,
                         int gate_pitch, int ones) {
    const int vdim = vdim_in + ones;                                         // columns of the state and of the output
    constexpr int PARTS = GLA_SPLIT * GLA_WARPS;
    constexpr int CH = DIMC / PARTS;                                         // channels per thread
    constexpr int BCOLS = GLA_BCOLS;                                         // columns per block
    static_assert(CH % 4 == 0 && GLA_COLS % (32 * GLA_WARPS) == 0, "whole float4s per thread; sets of four warps");
    extern __shared__ __align__(16) float gla_dyn[];
    float (*stage)[GROUP][3][DIMC] = reinterpret_cast<float (*)[GROUP][3][DIMC]>(gla_dyn);                 // [2]
    float (*stage_v)[GROUP][BCOLS] = reinterpret_cast<float (*)[GROUP][BCOLS]>(gla_dyn + 2 * GROUP * 3 * DIMC);   // [2]
    float (*partial)[GROUP][BCOLS][GLA_WARPS] =
        reinterpret_cast<float (*)[GROUP][BCOLS][GLA_WARPS]>(gla_dyn + 2 * GROUP * 3 * DIMC + 2 * GROUP * BCOLS);  // [2]
    constexpr int PER = (GROUP * DIMC + GLA_COLS - 1) / GLA_COLS;            // staged elements per thread and array
    constexpr int VPER = (GROUP * BCOLS + GLA_COLS - 1) / GLA_COLS;          // staged values per thread
    pdl_trigger();
    const int b = blockIdx.z, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wpart = warp % GLA_WARPS;                                      // this warp's share of the channels
    const int col = (warp / GLA_WARPS) * (32 / GLA_SPLIT) + lane / GLA_SPLIT, part = wpart * GLA_SPLIT + lane % GLA_SPLIT;
    const int j = blockIdx.x * BCOLS + col;
    const bool mine = j < vdim;
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    const int slot = seq_slot[b];
    float bs[PER];
#pragma unroll
    for (int e = 0; e < PER; e++) {
        const int d = (threadIdx.x + e * GLA_COLS) % DIMC;
        bs[e] = (d < dim && !gates) ? bias[h * dim + d] : 0.0f;
    }
    pdl_wait();
    float* st = state + ((size_t)slot * H + h) * dim * vdim;
    float S[CH];
#pragma unroll
    for (int i = 0; i < CH; i++) {
        const int d = (i / 4) * 4 * PARTS + 4 * part + (i & 3);
        S[i] = (mine && d < dim) ? st[(size_t)d * vdim + j] : 0.0f;
    }
    // as they come from memory (widened only when they are stored into a buffer, so that nothing waits for a load
    // before the group at hand has been computed)
    T rz[PER], rk[PER], rq[PER], rv[VPER];
    float ra[PER], rb[PER];                   // the second form's decay and key factor of the element's token
    auto fetch = [&](int base) {              // the raw values of tokens base .. base + GROUP - 1 into registers
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const int idx = threadIdx.x + e * GLA_COLS;
            const int g = idx / DIMC, d = idx % DIMC, t = base + g;
            rz[e] = rk[e] = rq[e] = T(0.0f);
            ra[e] = rb[e] = 1.0f;
            if (g < GROUP && t < t1 && d < dim) {
                const T* row = proj + (size_t)t * ld;
                if (gates) {
                    ra[e] = gates[((size_t)t * H + h) * gate_pitch];
                    rb[e] = gates[((size_t)t * H + h) * gate_pitch + 1];
                } else {
                    rz[e] = z[((size_t)t * H + h) * dim + d];
                }
                rk[e] = row[k_col + h * dim + d];
                rq[e] = row[q_col + h * dim + d];
            }
        }
        // the values: thread i takes token i / BCOLS of the group, column i % BCOLS (and so on, GLA_COLS further)
#pragma unroll
        for (int e = 0; e < VPER; e++) {
            const int idx = threadIdx.x + e * GLA_COLS;
            const int g = idx / BCOLS, jj = blockIdx.x * BCOLS + idx % BCOLS;
            rv[e] = T(0.0f);
            if (g < GROUP && base + g < t1 && jj < vdim_in) rv[e] = proj[(size_t)(base + g) * ld + v_col + h * vdim_in + jj];
            else if (g < GROUP && base + g < t1 && jj < vdim) rv[e] = T(1.0f);          // the column of ones
        }
    };
    auto store = [&](int buf, int base) {     // ... and from there into a buffer
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const int idx = threadIdx.x + e * GLA_COLS;
            const int g = idx / DIMC, d = idx % DIMC;
            if (g < GROUP) {
                // a token past the sequence's end: decay 1, key 0 (the state stays); a channel past dim: all zero
                const bool live = base + g < t1;
                stage[buf][g][0][d] = d < dim ? (live ? (gates ? ra[e] : gla_decay(ld_f(&rz[e]) + bs[e], inv_tau)) : 1.0f) : 0.0f;
                stage[buf][g][1][d] = gates ? ld_f(&rk[e]) * rb[e] : ld_f(&rk[e]);
                stage[buf][g][2][d] = ld_f(&rq[e]) * qscale;
            }
        }
#pragma unroll
        for (int e = 0; e < VPER; e++) {
            const int idx = threadIdx.x + e * GLA_COLS;
            if (idx < GROUP * BCOLS) stage_v[buf][idx / BCOLS][idx % BCOLS] = ld_f(&rv[e]);
        }
    };
    auto reduce = [&](int buf, int base) {    // a group's outputs: the four warps' sums in warp order
#pragma unroll
        for (int e = 0; e < VPER; e++) {
            const int idx = threadIdx.x + e * GLA_COLS;
            if (idx < GROUP * BCOLS) {
                const int g = idx / BCOLS, c = idx % BCOLS, jj = blockIdx.x * BCOLS + c;
                float acc = partial[buf][g][c][0];
#pragma unroll
                for (int w = 1; w < GLA_WARPS; w++) acc += partial[buf][g][c][w];
                if (jj < vdim && base + g < t1) o[((size_t)(base + g) * H + h) * vdim + jj] = acc;
            }
        }
    };
    fetch(t0);
    store(0, t0);
    __syncthreads();
    int buf = 0;
    for (int base = t0; base < t1; base += GROUP) {
        const bool more = base + GROUP < t1;
        if (more) fetch(base + GROUP);
        float acc[GROUP], vv[GROUP];
#pragma unroll
        for (int g = 0; g < GROUP; g++) {
            acc[g] = 0.0f;
            vv[g] = stage_v[buf][g][col];
        }
#pragma unroll
        for (int c = 0; c < CH / 4; c++) {
#pragma unroll
            for (int g = 0; g < GROUP; g++) {
                const int at = (c * PARTS + part) * 4;
                const float4 a = *reinterpret_cast<const float4*>(&stage[buf][g][0][at]);
                const float4 k = *reinterpret_cast<const float4*>(&stage[buf][g][1][at]);
                const float4 q = *reinterpret_cast<const float4*>(&stage[buf][g][2][at]);
                S[4 * c] = fmaf(a.x, S[4 * c], k.x * vv[g]);
                acc[g] = fmaf(S[4 * c], q.x, acc[g]);
                S[4 * c + 1] = fmaf(a.y, S[4 * c + 1], k.y * vv[g]);
                acc[g] = fmaf(S[4 * c + 1], q.y, acc[g]);
                S[4 * c + 2] = fmaf(a.z, S[4 * c + 2], k.z * vv[g]);
                acc[g] = fmaf(S[4 * c + 2], q.z, acc[g]);
                S[4 * c + 3] = fmaf(a.w, S[4 * c + 3], k.w * vv[g]);
                acc[g] = fmaf(S[4 * c + 3], q.w, acc[g]);
            }
        }
#pragma unroll
        for (int g = 0; g < GROUP; g++) {
            acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], 1);
            acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], 2);
            if (lane % GLA_SPLIT == 0) partial[buf][g][col][wpart] = acc[g];
        }
        if (more) store(buf ^ 1, base + GROUP);
        __syncthreads();              // the next group is staged, this one's partial sums are written
        reduce(buf, base);            // (the next group writes the other buffer of partial sums)
        buf ^= 1;
    }
    if (mine) {
#pragma unroll
        for (int i = 0; i < CH; i++) {
            const int d = (i / 4) * 4 * PARTS + 4 * part + (i & 3);
            if (d < dim) st[(size_t)d * vdim + j] = S[i];
        }
    }
}

// Any number of key channels: the state tile [dim][GLA_TILE] lives in shared memory.
template <typename T>
__global__ void __launch_bounds__(GLA_TILE)
gla_recurrent_kernel(const T* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, const T* __restrict__ z,
                     const float* __restrict__ bias, float inv_tau, float qscale, float* __restrict__ state,
                     float* __restrict__ o, const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int H,
                     int dim, int vdim_in, const float* __restrict__ gates, int gate_pitch, int ones) {
    const int vdim = vdim_in + ones;
    extern __shared__ float gla_smem[];
    float* S = gla_smem;                              // [dim][GLA_TILE]
    float* tok = S + (size_t)dim * GLA_TILE;          // two buffers of [3][dim]: decay, key, query
    pdl_trigger();
    const int b = blockIdx.z, h = blockIdx.y;
    const int j = blockIdx.x * GLA_TILE + threadIdx.x;
    const bool mine = j < vdim;
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    const int slot = seq_slot[b];
    pdl_wait();
    float* st = state + ((size_t)slot * H + h) * dim * vdim;
    for (int d = 0; d < dim; d++) S[d * GLA_TILE + threadIdx.x] = mine ? st[(size_t)d * vdim + j] : 0.0f;
    for (int t = t0; t < t1; t++) {
        float* cur = tok + (size_t)((t - t0) & 1) * 3 * dim;
        const T* row = proj + (size_t)t * ld;
        const float ga = gates ? gates[((size_t)t * H + h) * gate_pitch] : 1.0f;
        const float gb = gates ? gates[((size_t)t * H + h) * gate_pitch + 1] : 1.0f;
        for (int d = threadIdx.x; d < dim; d += GLA_TILE) {
            cur[d] = gates ? ga : gla_decay(ld_f(z + ((size_t)t * H + h) * dim + d) + bias[h * dim + d], inv_tau);
            cur[dim + d] = gates ? ld_f(row + k_col + h * dim + d) * gb : ld_f(row + k_col + h * dim + d);
            cur[2 * dim + d] = ld_f(row + q_col + h * dim + d) * qscale;
        }
        const float v = !mine ? 0.0f : (j < vdim_in ? ld_f(row + v_col + h * vdim_in + j) : 1.0f);
        __syncthreads();              // the token's vectors are there (the other buffer is free again after this barrier)
        float acc = 0.0f;
        for (int d = 0; d < dim; d++) {
            const float s = fmaf(cur[d], S[d * GLA_TILE + threadIdx.x], cur[dim + d] * v);
            S[d * GLA_TILE + threadIdx.x] = s;
            acc = fmaf(s, cur[2 * dim + d], acc);
        }
        if (mine) o[((size_t)t * H + h) * vdim + j] = acc;
    }
    if (mine)
        for (int d = 0; d < dim; d++) st[(size_t)d * vdim + j] = S[d * GLA_TILE + threadIdx.x];
}

static int gla_recurrent_go(const void* proj, long long ld, int q_col, int k_col, int v_col, const void* z,
                            const float* bias, float tau, float qscale, float* state, float* o, const int* seq_slot,
                            const int* seq_start, int seqs, int H, int dim, int vdim_in, int single, int dtype,
                            const float* gates, int gate_pitch, int ones, cudaStream_t stream) {
    // single: every sequence brings one token (a smaller staging group; the same results)
    if (seqs == 0) return 0;
    const int vdim = vdim_in + ones;                 // what the grid covers
    RI_REQUIRE(seqs > 0 && H > 0 && dim > 0 && vdim_in > 0 && tau > 0.0f, "gla_recurrent: bad sizes");
    RI_REQUIRE(gates ? gate_pitch >= 2 : (z && bias && !ones), "gla_recurrent: a decay per channel (z, bias) or per token (gates)");
    RI_REQUIRE(seqs <= 65535 && H <= 65535, "gla_recurrent: %d sequences, %d heads: too many for one launch", seqs, H);
    RI_REQUIRE(dtype == RI_DTYPE_F32 || dtype == RI_DTYPE_BF16, "gla_recurrent: unknown dtype %d", dtype);
    if (dim <= 128) {
        const int threads = GLA_COLS;             // all of them stage the tokens, whatever the number of columns
        const dim3 grid((vdim + GLA_BCOLS - 1) / GLA_BCOLS, H, seqs);
#define GLA_REG1(T, DIMC, GROUP)                                                                                           \
        do {                                                                                                               \
            const size_t sm = (size_t)(2 * GROUP * 3 * DIMC + 2 * GROUP * GLA_BCOLS * (1 + GLA_WARPS)) * sizeof(float);    \
            cudaError_t e = sm > 48 * 1024 ? cudaFuncSetAttribute(gla_recurrent_reg_kernel<T, DIMC, GROUP>,                \
                                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)   \
                                           : cudaSuccess;                                                                  \
            if (e != cudaSuccess) RI_FAIL((int)e, "gla_recurrent: %s", cudaGetErrorString(e));                             \
            ri_launch_pdl(gla_recurrent_reg_kernel<T, DIMC, GROUP>, grid, dim3(threads), sm, stream, (const T*)proj, ld,   \
                          q_col, k_col, v_col, (const T*)z, bias, 1.0f / tau, qscale, state, o, seq_slot, seq_start, H,    \
                          dim, vdim_in, gates, gate_pitch, ones);                                                          \
        } while (0)
    // tokens staged together: many, so that a trip to memory is paid once per 32 (16) tokens
#define GLA_REG(T, DIMC)                                                                                                   \
        do {                                                                                                               \
            if (single) GLA_REG1(T, DIMC, 1);                                                                              \
            else GLA_REG1(T, DIMC, (DIMC > 64 ? 16 : 32));                                                                 \
        } while (0)
#define GLA_BY_DIM(T)                                                                                                      \
        do {                                                                                                               \
            if (dim <= 64) GLA_REG(T, 64);                                                                                 \
            else GLA_REG(T, 128);                                                                                          \
        } while (0)
        if (dtype == RI_DTYPE_F32) GLA_BY_DIM(float);
        else GLA_BY_DIM(__nv_bfloat16);
#undef GLA_BY_DIM
#undef GLA_REG
#undef GLA_REG1
        RI_CHECK_LAUNCH("gla_recurrent");
        return 0;
    }
    const size_t smem = ((size_t)dim * GLA_TILE + 6 * (size_t)dim) * sizeof(float);
    RI_REQUIRE(smem <= 200 * 1024, "gla_recurrent: %d key channels per head do not fit in shared memory", dim);
    const dim3 grid((vdim + GLA_TILE - 1) / GLA_TILE, H, seqs);
    cudaError_t e = cudaSuccess;
#define GLA_GO(T)                                                                                                          \
    do {                                                                                                                   \
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(gla_recurrent_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) RI_FAIL((int)e, "gla_recurrent: %s", cudaGetErrorString(e));                                 \
        ri_launch_pdl(gla_recurrent_kernel<T>, grid, dim3(GLA_TILE), smem, stream, (const T*)proj, ld, q_col, k_col, v_col, \
                      (const T*)z, bias, 1.0f / tau, qscale, state, o, seq_slot, seq_start, H, dim, vdim_in, gates,        \
                      gate_pitch, ones);                                                                                   \
    } while (0)
    if (dtype == RI_DTYPE_F32) GLA_GO(float);
    else GLA_GO(__nv_bfloat16);
#undef GLA_GO
    RI_CHECK_LAUNCH("gla_recurrent");
    return 0;
}

extern "C" int ri_gla_recurrent(const void* proj, long long ld, int q_col, int k_col, int v_col, const void* z,
                                const float* bias, float tau, float qscale, float* state, float* o, const int* seq_slot,
                                const int* seq_start, int seqs, int H, int dim, int vdim, int single, int dtype,
                                cudaStream_t stream) {
    return gla_recurrent_go(proj, ld, q_col, k_col, v_col, z, bias, tau, qscale, state, o, seq_slot, seq_start, seqs, H, dim,
                            vdim, single, dtype, nullptr, 0, 0, stream);
}

// The second form: gates [tokens, H, gate_pitch] float32 with the decay at [0] and the key's factor at [1]; ones: the
// state [slots, H, dim, vdim + 1] and the output [tokens, H, vdim + 1] carry the column of ones.
extern "C" int ri_gla_recurrent_scalar(const void* proj, long long ld, int q_col, int k_col, int v_col, const float* gates,
                                       int gate_pitch, int ones, float qscale, float* state, float* o, const int* seq_slot,
                                       const int* seq_start, int seqs, int H, int dim, int vdim, int single, int dtype,
                                       cudaStream_t stream) {
    RI_REQUIRE(gates != nullptr && (ones == 0 || ones == 1), "gla_recurrent_scalar: gates are needed");
    return gla_recurrent_go(proj, ld, q_col, k_col, v_col, nullptr, nullptr, 1.0f, qscale, state, o, seq_slot, seq_start, seqs,
                            H, dim, vdim, single, dtype, gates, gate_pitch, ones, stream);
}

// y[t, h, j] = T( o[t, h, j] / sqrt(mean_j o[t, h, :]^2 + eps) * gain[j] * f(g[t, h vdim + j]) ),  f: silu (fn 1) or
// sigmoid (fn 0); a warp per (token, head), the sum of squares over the warp's tree.
template <typename T>
__global__ void gla_head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gain, float eps,
                                          const T* __restrict__ g, long long ldg, T* __restrict__ y, int H, int vdim,
                                          int fn, size_t units) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const size_t unit = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= units) return;
    const size_t t = unit / H;
    const int h = (int)(unit - t * H);
    const float* op = o + unit * vdim;
    float ss = 0.0f;
    for (int j = lane; j < vdim; j += 32) ss += op[j] * op[j];
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    for (int j = lane; j < vdim; j += 32) {
        const float zg = ld_f(g + t * ldg + (size_t)h * vdim + j);
        const float s = 1.0f / (1.0f + expf(-zg));
        st_f(y + unit * vdim + j, op[j] * inv * gain[j] * (fn == 1 ? zg * s : s));
    }
}

extern "C" int ri_gla_head_norm_gate(const float* o, const float* gain, float eps, const void* g, long long ldg, void* y,
                                     int tokens, int H, int vdim, int fn, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(tokens > 0 && H > 0 && vdim > 0, "gla_head_norm_gate: bad sizes");
    const size_t units = (size_t)tokens * H;
    const unsigned blocks = (unsigned)((units + 7) / 8);
    if (dtype == RI_DTYPE_F32)
        ri_launch_pdl(gla_head_norm_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, o, gain, eps, (const float*)g, ldg, (float*)y, H, vdim, fn, units);
    else if (dtype == RI_DTYPE_BF16)
        ri_launch_pdl(gla_head_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, o, gain, eps, (const __nv_bfloat16*)g, ldg, (__nv_bfloat16*)y, H, vdim, fn, units);
    else RI_FAIL(-1, "gla_head_norm_gate: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("gla_head_norm_gate");
    return 0;
}
