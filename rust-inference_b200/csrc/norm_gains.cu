// RMS norm of a single-stream float32 residual with one or two gains, and everything that joins the residual in
// front of it, in one pass over the row.
//
// resid [n, dim] float32.  One block per output row does, element by element and in this order:
//   1. the outputs that the layer before left pending (compute type T, up to two, each with an optional float32
//      factor w[0]):  one output  x' = x + w1 y1;  two  x' = x + (w1 y1 + w2 y2)   (the outputs' sum first);
//      with a norm behind the sublayer (`post_gain`, float32 [dim]) the sum s = w1 y1 (+ w2 y2) is normed before it
//      joins:  x' = x + s / sqrt(mean(s^2) + post_eps) * post_gain   (the gain holds the layer's scale as well);
//   2. the terms of a pass's entry: x' += float(table[ids[row]]) * scale   (the embedding's row once more; ids null: not),
//      then x' += vec   (a learned vector; null: not);
//      x' is written back to resid, unless only some rows are read (`rows`: nothing reads resid after that call);
//   3. r = 1 / sqrt(mean(x'^2) + eps);  out1 = x' r gain1  and, with a second gain, out2 = x' r gain2.
//      Without gain1 nothing is normed: out1 (if given) gets x' itself in the compute type, its rows `out_pitch`
//      elements apart (the left half of a wider matrix that a product reads next).
// A layer whose mixer and feed-forward both read the same residual, each through a norm of its own, needs the
// statistic once and the residual read once; that is what the second gain is for.
// All arithmetic is float32 whatever T is.  The block size and the order of a row's additions depend on dim (and on
// the pointers' alignment) only, never on how many rows a step has: a row's result is the same bits in any batch.
#include "common.cuh"
#include "linear_skinny_geometry.cuh"

__device__ __forceinline__ float4 ng_ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ng_ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void ng_st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void ng_st4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const unsigned*>(&a);
    u.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

struct NgArgs {
    float* resid;
    const void *y1, *y2, *table;
    const float *w1, *w2, *vec, *gain1, *gain2;
    const int *ids, *rows;
    void *out1, *out2;
    int dim, vocab, write_back;
    float scale, eps;
    int* err;
    const float* post_gain;
    float post_eps;
    long long out_pitch;
    int n_rows;          // blocks past the rows ask for the weights that the linear after this norm reads first
    WeightHint next;
};

// one element's new value; `e` is its index in the row
template <typename T>
__device__ __forceinline__ float ng_join(float x, const T* y1, const T* y2, float w1, float w2, const T* trow, float scale,
                                         const float* vec, int e) {
    if (y2) x = x + (w1 * ld_f(y1 + e) + w2 * ld_f(y2 + e));
    else if (y1) x = x + w1 * ld_f(y1 + e);
    if (trow) x = x + ld_f(trow + e) * scale;
    if (vec) x = x + vec[e];
    return x;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(512) norm_gains_kernel(NgArgs a) {
    extern __shared__ __align__(16) float ng_row[];                 // [dim]
    __shared__ float red[33];
    pdl_trigger();
    // parameters and the step's tables are not written by the kernel in front: read before the wait for it
    const float w1 = a.w1 ? a.w1[0] : 1.0f, w2 = a.w2 ? a.w2[0] : 1.0f;
    const bool hint_block = (int)blockIdx.x >= a.n_rows;
    const size_t r = (a.rows && !hint_block) ? (size_t)a.rows[blockIdx.x] : (size_t)blockIdx.x;
    const T* trow = nullptr;
    if (a.ids && !hint_block) {
        const int id = a.ids[r];
        if (id < 0 || id >= a.vocab) {
            if (threadIdx.x == 0) atomicExch(a.err, 1);             // a token outside the table: its row is not added
        } else {
            trow = (const T*)a.table + (size_t)id * a.dim;
        }
    }
    pdl_wait();
    if (hint_block) {
        weight_hint_prefetch(a.next, ((int)blockIdx.x - a.n_rows) * (int)blockDim.x + (int)threadIdx.x,
                             ((int)gridDim.x - a.n_rows) * (int)blockDim.x);
        return;
    }
    const int dim = a.dim;
    float* rp = a.resid + r * dim;
    const T* y1 = a.y1 ? (const T*)a.y1 + r * dim : nullptr;
    const T* y2 = (a.y1 && a.y2) ? (const T*)a.y2 + r * dim : nullptr;
    const bool changes = y1 || trow || a.vec;
    const bool post = y1 && a.post_gain;
    float sum = 0.0f;
    float pinv = 1.0f;
    if (post) {
        // the pending outputs' sum, normed on its own before it joins: the sum waits in the row buffer
        float ss = 0.0f;
        if (VEC) {
            for (int i = threadIdx.x; i < (dim >> 2); i += blockDim.x) {
                const float4 p1 = ng_ld4(y1 + 4 * i);
                float4 s4 = make_float4(w1 * p1.x, w1 * p1.y, w1 * p1.z, w1 * p1.w);
                if (y2) {
                    const float4 p2 = ng_ld4(y2 + 4 * i);
                    s4 = make_float4(s4.x + w2 * p2.x, s4.y + w2 * p2.y, s4.z + w2 * p2.z, s4.w + w2 * p2.w);
                }
                *reinterpret_cast<float4*>(ng_row + 4 * i) = s4;
                ss += (s4.x * s4.x + s4.y * s4.y) + (s4.z * s4.z + s4.w * s4.w);
            }
        } else {
            for (int i = threadIdx.x; i < dim; i += blockDim.x) {
                float v = w1 * ld_f(y1 + i);
                if (y2) v = v + w2 * ld_f(y2 + i);
                ng_row[i] = v;
                ss += v * v;
            }
        }
        pinv = 1.0f / sqrtf(block_sum(ss, red) / (float)dim + a.post_eps);
    }
    if (VEC) {
        for (int i = threadIdx.x; i < (dim >> 2); i += blockDim.x) {
            float4 x = ng_ld4(rp + 4 * i);
            if (changes) {
                float4 p1 = make_float4(0.f, 0.f, 0.f, 0.f), p2 = p1, tr = p1, vv = p1;
                if (post) {
                    const float4 s4 = *reinterpret_cast<const float4*>(ng_row + 4 * i);
                    const float4 pg = ng_ld4(a.post_gain + 4 * i);
                    x.x = x.x + s4.x * pinv * pg.x; x.y = x.y + s4.y * pinv * pg.y;
                    x.z = x.z + s4.z * pinv * pg.z; x.w = x.w + s4.w * pinv * pg.w;
                } else {
                    if (y1) p1 = ng_ld4(y1 + 4 * i);
                    if (y2) p2 = ng_ld4(y2 + 4 * i);
                }
                if (trow) tr = ng_ld4(trow + 4 * i);
                if (a.vec) vv = ng_ld4(a.vec + 4 * i);
                if (post) {
                } else if (y2) {
                    x.x = x.x + (w1 * p1.x + w2 * p2.x); x.y = x.y + (w1 * p1.y + w2 * p2.y);
                    x.z = x.z + (w1 * p1.z + w2 * p2.z); x.w = x.w + (w1 * p1.w + w2 * p2.w);
                } else if (y1) {
                    x.x = x.x + w1 * p1.x; x.y = x.y + w1 * p1.y; x.z = x.z + w1 * p1.z; x.w = x.w + w1 * p1.w;
                }
                if (trow) { x.x = x.x + tr.x * a.scale; x.y = x.y + tr.y * a.scale; x.z = x.z + tr.z * a.scale; x.w = x.w + tr.w * a.scale; }
                if (a.vec) { x.x = x.x + vv.x; x.y = x.y + vv.y; x.z = x.z + vv.z; x.w = x.w + vv.w; }
                if (a.write_back) ng_st4(rp + 4 * i, x);
            }
            *reinterpret_cast<float4*>(ng_row + 4 * i) = x;
            sum += (x.x * x.x + x.y * x.y) + (x.z * x.z + x.w * x.w);
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            float x = rp[i];
            if (changes) {
                if (post) {
                    x = x + ng_row[i] * pinv * a.post_gain[i];
                    x = ng_join<T>(x, nullptr, nullptr, w1, w2, trow, a.scale, a.vec, i);
                } else {
                    x = ng_join<T>(x, y1, y2, w1, w2, trow, a.scale, a.vec, i);
                }
                if (a.write_back) rp[i] = x;
            }
            ng_row[i] = x;
            sum += x * x;
        }
    }
    if (!a.gain1) {
        // nothing is normed: the new residual itself, in the compute type, for whoever reads it next
        if (a.out1) {
            __syncthreads();
            T* oc = (T*)a.out1 + (size_t)blockIdx.x * a.out_pitch;
            for (int i = threadIdx.x; i < dim; i += blockDim.x) st_f(oc + i, ng_row[i]);
        }
        return;
    }
    const float inv = 1.0f / sqrtf(block_sum(sum, red) / (float)dim + a.eps);
    T* o1 = (T*)a.out1 + (size_t)blockIdx.x * dim;
    T* o2 = a.out2 ? (T*)a.out2 + (size_t)blockIdx.x * dim : nullptr;
    if (VEC) {
        for (int i = threadIdx.x; i < (dim >> 2); i += blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(ng_row + 4 * i);
            const float4 g = ng_ld4(a.gain1 + 4 * i);
            ng_st4(o1 + 4 * i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
            if (o2) {
                const float4 h = ng_ld4(a.gain2 + 4 * i);
                ng_st4(o2 + 4 * i, make_float4(v.x * inv * h.x, v.y * inv * h.y, v.z * inv * h.z, v.w * inv * h.w));
            }
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            const float v = ng_row[i];
            st_f(o1 + i, v * inv * a.gain1[i]);
            if (o2) st_f(o2 + i, v * inv * a.gain2[i]);
        }
    }
}

// y1/w1, y2/w2: pending outputs [n, dim] of type `dtype` and their float32 factors (null: 1); ids/table/vocab/scale, vec:
// the entry terms (each may be null); rows: int32 indices of the rows to read (null: all n_rows, with write-back);
// gain2/out2 may be null.  next_w [next_n, next_k] (bfloat16, or null): the weights of the weight-streaming linear that
// reads the first result; the kernel asks for the part of them that the linear wants first after what it holds itself
// (a hint: it changes no result).
extern "C" int ri_norm_gains(float* resid, const void* y1, const float* w1, const void* y2, const float* w2, const int* ids,
                             const void* table, int vocab, float scale, const float* vec, const int* rows,
                             const float* gain1, const float* gain2, void* out1, void* out2, int n_rows, int dim, float eps,
                             int dtype, const void* next_w, int next_n, int next_k, int* err_flag, cudaStream_t stream);

// The same with a norm behind the pending outputs (post_gain [dim] float32 or null, post_eps) and, when gain1 is null,
// no norm in front: out1 (or null) then gets the new residual in the compute type at rows `out_pitch` elements apart.
extern "C" int ri_norm_gains_post(float* resid, const void* y1, const float* w1, const void* y2, const float* w2, const int* ids,
                                  const void* table, int vocab, float scale, const float* vec, const int* rows,
                                  const float* gain1, const float* gain2, void* out1, void* out2, int n_rows, int dim,
                                  float eps, const float* post_gain, float post_eps, long long out_pitch, int dtype,
                                  const void* next_w, int next_n, int next_k, int* err_flag, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    RI_REQUIRE(n_rows > 0 && dim > 0, "norm_gains: bad sizes rows=%d dim=%d", n_rows, dim);
    RI_REQUIRE(dtype == RI_DTYPE_F32 || dtype == RI_DTYPE_BF16, "norm_gains: unknown dtype %d", dtype);
    RI_REQUIRE(y1 || !y2, "norm_gains: pending outputs are given first, second");
    RI_REQUIRE((gain2 == nullptr) == (out2 == nullptr), "norm_gains: a second gain and a second output go together");
    RI_REQUIRE(gain1 || (!gain2 && !next_w), "norm_gains: without a first gain nothing is normed");
    RI_REQUIRE(gain1 ? out1 != nullptr : (!out1 || out_pitch >= dim), "norm_gains: bad output for %d columns", dim);
    RI_REQUIRE(!post_gain || y1, "norm_gains: a norm behind the sublayer needs its output");
    RI_REQUIRE(!ids || (table && vocab > 0), "norm_gains: token ids need the table");
    RI_REQUIRE(!ids || !rows, "norm_gains: the entry terms join whole steps, not selected rows");
    const size_t smem = (size_t)dim * sizeof(float);
    RI_REQUIRE(smem <= 200 * 1024, "norm_gains: a row of %d elements does not fit in shared memory (limit 51200)", dim);
    NgArgs a;
    a.resid = resid; a.y1 = y1; a.y2 = y2; a.table = ids ? table : nullptr; a.w1 = w1; a.w2 = w2; a.vec = vec;
    a.gain1 = gain1; a.gain2 = gain2; a.ids = ids; a.rows = rows; a.out1 = out1; a.out2 = out2; a.dim = dim; a.vocab = vocab;
    a.write_back = rows ? 0 : 1; a.scale = scale; a.eps = eps; a.err = err_flag;
    a.post_gain = post_gain; a.post_eps = post_eps; a.out_pitch = out_pitch;
    a.n_rows = n_rows;
    a.next = make_weight_hint(nullptr, 0, 0, 0);
    if (next_w) {
        static int sms = 0;
        if (!sms) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        }
        a.next = make_weight_hint(next_w, next_n, next_k, sms);
    }
    const uintptr_t unit = dtype == RI_DTYPE_F32 ? 15 : 7;
    const bool vec4 = dim % 4 == 0 && (((uintptr_t)resid | (uintptr_t)gain1 | (uintptr_t)gain2 | (uintptr_t)vec | (uintptr_t)post_gain) & 15) == 0 &&
                      (((uintptr_t)y1 | (uintptr_t)y2 | (uintptr_t)table | (uintptr_t)out1 | (uintptr_t)out2) & unit) == 0;
    // by the row length alone: the order of a row's additions must not depend on how many rows the step has
    int threads;
    if (vec4) {
        const int nvec = dim / 4;
        threads = nvec >= 256 ? 256 : ((nvec + 31) / 32) * 32;
    } else {
        threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
    }
    // with a hint: as many more blocks as give each thread a few requests
    int extra = 0;
    if (a.next.base) {
        const long long lines = (long long)a.next.rows * SK_WARPS * (SK_HINT_STAGES * SK_STAGE_K * 2 / SK_HINT_LINE);
        const int want = (int)((lines + (long long)threads * 2 - 1) / ((long long)threads * 2));
        extra = want < 1 ? 1 : (want > 256 ? 256 : want);
    }
    cudaError_t e = cudaSuccess;
#define NG_GO(T, V)                                                                                                      \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            e = cudaFuncSetAttribute(norm_gains_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        if (e != cudaSuccess) RI_FAIL((int)e, "norm_gains: %s", cudaGetErrorString(e));                                  \
        ri_launch_pdl(norm_gains_kernel<T, V>, dim3(n_rows + extra), dim3(threads), smem, stream, a);                           \
    } while (0)
    if (dtype == RI_DTYPE_F32) {
        if (vec4) NG_GO(float, true); else NG_GO(float, false);
    } else {
        if (vec4) NG_GO(__nv_bfloat16, true); else NG_GO(__nv_bfloat16, false);
    }
#undef NG_GO
    RI_CHECK_LAUNCH("norm_gains");
    return 0;
}

extern "C" int ri_norm_gains(float* resid, const void* y1, const float* w1, const void* y2, const float* w2, const int* ids,
                             const void* table, int vocab, float scale, const float* vec, const int* rows,
                             const float* gain1, const float* gain2, void* out1, void* out2, int n_rows, int dim, float eps,
                             int dtype, const void* next_w, int next_n, int next_k, int* err_flag, cudaStream_t stream) {
    return ri_norm_gains_post(resid, y1, w1, y2, w2, ids, table, vocab, scale, vec, rows, gain1, gain2, out1, out2, n_rows, dim,
                              eps, nullptr, 0.0f, 0, dtype, next_w, next_n, next_k, err_flag, stream);
}
