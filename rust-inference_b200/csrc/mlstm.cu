// The matrix memory of xLSTM (mLSTM): what stands around the recurrence over the state.
//
// Per token t and head, from the pre-activations zi, zf of the input and forget gates (columns of a projection):
//   li = cap tanh((zi + bi) / cap)                         log input gate
//   lf = log_sigmoid(cap tanh((zf + bf) / cap))            log forget gate
//   m_t = max(lf + m_(t-1), li)                            running maximum, m = 0 at a sequence's start
//   a_t = exp(lf + m_(t-1) - m_t),  b_t = exp(li - m_t)    what the state is decayed by, and what the key is scaled by
//   S_t = a_t S_(t-1) + b_t k_t v_t^T,  n_t = a_t n_(t-1) + b_t k_t        (the recurrence kernel of gla.cu, second form,
//                                                                            with n as one more column of S)
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//   y_t = o_t / sqrt(mean_j(o_t[j]^2) + eps) * gain[h, j] * sigmoid(g_t[h, j])        per head
//
// `mlstm_gates`: a warp per (sequence, head) walks the step's new tokens 32 at a time: every lane takes one token's li
// and lf (the transcendental functions, in parallel), then all lanes run the chain m_t = max(lf + m, li) over the 32
// tokens in order, and every lane writes its token's (a, b, exp(-m)).  m is read from and written back to the
// sequence's slot of `m_state` [slots, H].  The chain is the same whatever the cutting of the sequence into steps, so
// prompts, pieces and single tokens give the same bits.  All float32 with full-precision functions.
//
// `mlstm_head_norm_gate`: a warp per (token, head) reads the recurrence's output row [vdim + 1] (the last element is
// n . q), divides, norms, applies gain and gate and writes the compute type.
#include "common.cuh"

#define ML_WARPS 4

__device__ __forceinline__ float ml_log_sigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

template <typename T>
__global__ void __launch_bounds__(32 * ML_WARPS)
mlstm_gates_kernel(const T* __restrict__ proj, long long ld, int i_col, int f_col, const float* __restrict__ i_bias,
                   const float* __restrict__ f_bias, float cap, float* __restrict__ m_state, float* __restrict__ gates,
                   const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int H) {
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int h = blockIdx.x * ML_WARPS + (threadIdx.x >> 5);
    const int b = blockIdx.y;
    if (h >= H) return;
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    const int slot = seq_slot[b];
    const float bi = i_bias[h], bf = f_bias[h];
    pdl_wait();
    float m = m_state[(size_t)slot * H + h];
    for (int base = t0; base < t1; base += 32) {
        const int t = base + lane;
        float li = 0.0f, lf = 0.0f;
        if (t < t1) {
            const T* row = proj + (size_t)t * ld;
            li = cap * tanhf((ld_f(row + i_col + h) + bi) / cap);
            lf = ml_log_sigmoid(cap * tanhf((ld_f(row + f_col + h) + bf) / cap));
        }
        float m_before = 0.0f, m_mine = 0.0f;
        const int n = min(32, t1 - base);
        for (int g = 0; g < n; g++) {
            const float lfg = __shfl_sync(0xffffffffu, lf, g), lig = __shfl_sync(0xffffffffu, li, g);
            const float m_new = fmaxf(lfg + m, lig);
            if (lane == g) {
                m_before = m;
                m_mine = m_new;
            }
            m = m_new;
        }
        if (t < t1) {
            float* out = gates + ((size_t)t * H + h) * 3;
            out[0] = expf(lf + m_before - m_mine);
            out[1] = expf(li - m_mine);
            out[2] = expf(-m_mine);
        }
    }
    if (lane == 0) m_state[(size_t)slot * H + h] = m;
}

// The same for prompts: a block of ML_BLOCK threads per (sequence, head) takes ML_BLOCK tokens at a time: every thread its
// token's li and lf, then ONE thread the chain over them from shared memory (the same operations in the same order as in
// the kernel above: the same bits), then every thread its token's three results.
#define ML_BLOCK 256
template <typename T>
__global__ void __launch_bounds__(ML_BLOCK)
mlstm_gates_block_kernel(const T* __restrict__ proj, long long ld, int i_col, int f_col, const float* __restrict__ i_bias,
                         const float* __restrict__ f_bias, float cap, float* __restrict__ m_state, float* __restrict__ gates,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int H) {
    __shared__ __align__(16) float s_li[ML_BLOCK], s_lf[ML_BLOCK], s_before[ML_BLOCK], s_mine[ML_BLOCK];
    __shared__ float s_m;
    pdl_trigger();
    const int h = blockIdx.x, b = blockIdx.y;
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    const int slot = seq_slot[b];
    const float bi = i_bias[h], bf = f_bias[h];
    pdl_wait();
    if (threadIdx.x == 0) s_m = m_state[(size_t)slot * H + h];
    for (int base = t0; base < t1; base += ML_BLOCK) {
        const int t = base + threadIdx.x;
        float li = 0.0f, lf = 0.0f;
        if (t < t1) {
            const T* row = proj + (size_t)t * ld;
            li = cap * tanhf((ld_f(row + i_col + h) + bi) / cap);
            lf = ml_log_sigmoid(cap * tanhf((ld_f(row + f_col + h) + bf) / cap));
        }
        s_li[threadIdx.x] = li;
        s_lf[threadIdx.x] = lf;
        __syncthreads();
        if (threadIdx.x == 0) {
            // eight tokens' gates into registers at a time, so that only the additions and maxima form the chain
            float m = s_m;
            const int n = min(ML_BLOCK, t1 - base);
            for (int g0 = 0; g0 < n; g0 += 8) {
                const float4 fa = *reinterpret_cast<const float4*>(s_lf + g0), fb = *reinterpret_cast<const float4*>(s_lf + g0 + 4);
                const float4 ia = *reinterpret_cast<const float4*>(s_li + g0), ib = *reinterpret_cast<const float4*>(s_li + g0 + 4);
                const float f8[8] = {fa.x, fa.y, fa.z, fa.w, fb.x, fb.y, fb.z, fb.w};
                const float i8[8] = {ia.x, ia.y, ia.z, ia.w, ib.x, ib.y, ib.z, ib.w};
                float before[8], mine[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    // (tokens past the step's end hold li = lf = 0 and are computed too; their results are not read,
                    // and m is taken from the last real token below)
                    before[j] = m;
                    m = fmaxf(f8[j] + m, i8[j]);
                    mine[j] = m;
                }
                *reinterpret_cast<float4*>(s_before + g0) = make_float4(before[0], before[1], before[2], before[3]);
                *reinterpret_cast<float4*>(s_before + g0 + 4) = make_float4(before[4], before[5], before[6], before[7]);
                *reinterpret_cast<float4*>(s_mine + g0) = make_float4(mine[0], mine[1], mine[2], mine[3]);
                *reinterpret_cast<float4*>(s_mine + g0 + 4) = make_float4(mine[4], mine[5], mine[6], mine[7]);
            }
            s_m = s_mine[n - 1];
        }
        __syncthreads();
        if (t < t1) {
            const float m_before = s_before[threadIdx.x], m_mine = s_mine[threadIdx.x];
            float* out = gates + ((size_t)t * H + h) * 3;
            out[0] = expf(lf + m_before - m_mine);
            out[1] = expf(li - m_mine);
            out[2] = expf(-m_mine);
        }
        // (the next round's first barrier stands between these reads and the chain's next writes)
    }
    __syncthreads();
    if (threadIdx.x == 0) m_state[(size_t)slot * H + h] = s_m;
}

// proj [tokens, ld] of the type `dtype`; i and f pre-activations of head h at columns i_col + h and f_col + h;
// gates [tokens, H, 3] float32 out.
// single: every sequence brings one token (a warp per sequence and head); else a block per sequence and head.
extern "C" int ri_mlstm_gates(const void* proj, long long ld, int i_col, int f_col, const float* i_bias, const float* f_bias,
                              float cap, float* m_state, float* gates, const int* seq_slot, const int* seq_start, int seqs,
                              int H, int single, int dtype, cudaStream_t stream) {
    if (seqs == 0) return 0;
    RI_REQUIRE(seqs > 0 && seqs <= 65535 && H > 0 && cap > 0.0f, "mlstm_gates: bad sizes (seqs %d, heads %d, cap %g)", seqs, H, cap);
    if (!single) {
        const dim3 bgrid(H, seqs);
        if (dtype == RI_DTYPE_F32)
            ri_launch_pdl(mlstm_gates_block_kernel<float>, bgrid, dim3(ML_BLOCK), 0, stream, (const float*)proj, ld, i_col, f_col,
                          i_bias, f_bias, cap, m_state, gates, seq_slot, seq_start, H);
        else if (dtype == RI_DTYPE_BF16)
            ri_launch_pdl(mlstm_gates_block_kernel<__nv_bfloat16>, bgrid, dim3(ML_BLOCK), 0, stream, (const __nv_bfloat16*)proj, ld,
                          i_col, f_col, i_bias, f_bias, cap, m_state, gates, seq_slot, seq_start, H);
        else RI_FAIL(-1, "mlstm_gates: unknown dtype %d", dtype);
        RI_CHECK_LAUNCH("mlstm_gates");
        return 0;
    }
    const dim3 grid((H + ML_WARPS - 1) / ML_WARPS, seqs);
    if (dtype == RI_DTYPE_F32)
        ri_launch_pdl(mlstm_gates_kernel<float>, grid, dim3(32 * ML_WARPS), 0, stream, (const float*)proj, ld, i_col, f_col, i_bias,
                      f_bias, cap, m_state, gates, seq_slot, seq_start, H);
    else if (dtype == RI_DTYPE_BF16)
        ri_launch_pdl(mlstm_gates_kernel<__nv_bfloat16>, grid, dim3(32 * ML_WARPS), 0, stream, (const __nv_bfloat16*)proj, ld,
                      i_col, f_col, i_bias, f_bias, cap, m_state, gates, seq_slot, seq_start, H);
    else RI_FAIL(-1, "mlstm_gates: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("mlstm_gates");
    return 0;
}

template <typename TG, typename TY>
__global__ void mlstm_head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gates,
                                            const float* __restrict__ gain, float eps, const TG* __restrict__ g, long long ldg,
                                            TY* __restrict__ y, int H, int vdim, size_t units) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const size_t unit = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= units) return;
    const size_t t = unit / H;
    const int h = (int)(unit - t * H);
    const float* op = o + unit * (vdim + 1);
    const float den = fmaxf(fabsf(op[vdim]), gates[unit * 3 + 2]) + 1e-6f;
    float ss = 0.0f;
    for (int j = lane; j < vdim; j += 32) {
        const float v = op[j] / den;
        ss += v * v;
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    for (int j = lane; j < vdim; j += 32) {
        const float zg = ld_f(g + t * ldg + (size_t)h * vdim + j);
        const float s = 1.0f / (1.0f + expf(-zg));
        st_f(y + unit * vdim + j, op[j] / den * inv * gain[(size_t)h * vdim + j] * s);
    }
}

// o [tokens, H, vdim + 1] float32 (the last column is n . q), gates [tokens, H, 3] (exp(-m) at [2]), gain [H vdim] float32,
// g: the gate's pre-activations, columns of a matrix of type g_dtype with row pitch ldg; y [tokens, H vdim] of type y_dtype.
extern "C" int ri_mlstm_head_norm_gate(const float* o, const float* gates, const float* gain, float eps, const void* g,
                                       long long ldg, void* y, int tokens, int H, int vdim, int g_dtype, int y_dtype,
                                       cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(tokens > 0 && H > 0 && vdim > 0, "mlstm_head_norm_gate: bad sizes");
    const size_t units = (size_t)tokens * H;
    const unsigned blocks = (unsigned)((units + 7) / 8);
#define ML_GO(TG, TY)                                                                                                     \
    ri_launch_pdl(mlstm_head_norm_gate_kernel<TG, TY>, dim3(blocks), dim3(256), 0, stream, o, gates, gain, eps, (const TG*)g, \
                  ldg, (TY*)y, H, vdim, units)
    if (g_dtype == RI_DTYPE_F32 && y_dtype == RI_DTYPE_F32) ML_GO(float, float);
    else if (g_dtype == RI_DTYPE_F32 && y_dtype == RI_DTYPE_BF16) ML_GO(float, __nv_bfloat16);
    else if (g_dtype == RI_DTYPE_BF16 && y_dtype == RI_DTYPE_BF16) ML_GO(__nv_bfloat16, __nv_bfloat16);
    else RI_FAIL(-1, "mlstm_head_norm_gate: dtypes %d, %d", g_dtype, y_dtype);
#undef ML_GO
    RI_CHECK_LAUNCH("mlstm_head_norm_gate");
    return 0;
}
