// A routed feed-forward (mixture of experts): router, plan of the step, grouped products, combination.
//
// `moe_route`   per token: logits z = R x (float32), scores s = softmax(z) over all N outputs of the router (or the
//               sigmoid of each), choice scores s + correction, optionally only within the best groups of neighbouring
//               outputs (`MoeRule`), the `top` largest of them (ties: the lower index), and as weights the chosen
//               outputs' scores s divided by their sum (+ 1e-20) or as they are, times a constant.  Every sum has a
//               fixed order.
// `moe_plan`    the step's (token, choice) pairs grouped by expert: `perm` lists the pairs of expert 0, then of expert
//               1 and so on (pairs whose choice is not one of the first E outputs, identity experts, are left out), and
//               `tiles` cuts every expert's run into tiles of MOE_BM rows: (expert, first row in perm, rows).  One
//               block; which pair lands where inside an expert's run is not fixed, and no result depends on it: a
//               row of a product is computed alone.
// `moe_grouped_linear`  y[out(r), :] = W[e] a[in(r), :] for every row r of every tile, W [E, N, K]; in(r) = perm[r] /
//               div (gather: a token's row for each of its pairs) or r, out(r) = perm[r] (scatter: back to the pair's
//               own place) or r.  float32: FMA tiles, k ascending in one accumulator per output; bfloat16: mma.sync
//               m16n8k16 with float32 accumulators.  The grid covers the most tiles a step can have; blocks past the
//               plan's count leave at once (the count stays on the device: no trip to the host, and the step can be
//               replayed from a graph).
// `moe_combine` y[t] = sum_j w[t, j] (choice j an identity expert ? x[t] : pair_out[t top + j]) (+ extra[t]),
//               j ascending, float32, rounded once.
#include "common.cuh"
#include "mma_helpers.cuh"

#define MOE_BM 32
#define MOE_BM_WIDE 64
#define MOE_BN 64
#define MOE_ROUTE_WARPS 4

// A warp per token.  The logits are taken four router outputs at a time: a lane walks its own k (four neighbouring ones
// per trip with 16-byte loads where the rows allow it, else one) and keeps four sums, so that twenty loads are on their
// way together; a sum's order depends on the row's size alone.  Then the warp does the softmax and the choice.
__device__ __forceinline__ float4 moe_ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 moe_ld4(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

// How scores become a choice and weights.  mode 0: scores are the softmax over all outputs; mode 1: the sigmoid of every
// output on its own.  Choice scores are the scores plus the correction.  groups > 1: the outputs form `groups` equal runs
// of neighbours, a run's score is the sum of its `gtop` largest choice scores, and only the outputs of the `keep` best
// runs can be chosen (ties: the lower index, for runs as for outputs).  The weights are the chosen outputs' scores
// (without the correction) times `scale`, divided by their sum first when `renorm` is set.
struct MoeRule {
    int mode, groups, keep, gtop, renorm;
    float scale;
};

// One warp: s [N] holds the logits on entry, c [N] and gs [groups] are scratch.
__device__ __forceinline__ void moe_choose(float* s, float* c, float* gs, const float* __restrict__ correction,
                                           int* __restrict__ idx, float* __restrict__ weight, int t, int N, int top, int lane,
                                           const MoeRule rule) {
    if (rule.mode == 0) {
        float mx = -INFINITY;
        for (int n = lane; n < N; n += 32) mx = fmaxf(mx, s[n]);
        mx = warp_max(mx);
        float sum = 0.0f;
        for (int n = lane; n < N; n += 32) {
            const float e = expf(s[n] - mx);
            s[n] = e;
            sum += e;
        }
        sum = warp_sum(sum);
        for (int n = lane; n < N; n += 32) {
            s[n] = s[n] / sum;
            c[n] = s[n] + correction[n];
        }
    } else {
        for (int n = lane; n < N; n += 32) {
            s[n] = 1.0f / (1.0f + expf(-s[n]));
            c[n] = s[n] + correction[n];
        }
    }
    __syncwarp();
    if (rule.groups > 1) {
        const int size = N / rule.groups;
        for (int g = lane; g < rule.groups; g += 32) {
            // the gtop largest of the run, one after the other in the order (value descending, index ascending)
            float total = 0.0f, last = INFINITY;
            int last_at = -1;
            for (int r = 0; r < rule.gtop && r < size; r++) {
                float best = -INFINITY;
                int at = -1;
                for (int n = 0; n < size; n++) {
                    const float v = c[g * size + n];
                    const bool after = v < last || (v == last && n > last_at);
                    if (after && (at < 0 || v > best)) {
                        best = v;
                        at = n;
                    }
                }
                if (at < 0) break;
                total += best;
                last = best;
                last_at = at;
            }
            gs[g] = total;
        }
        __syncwarp();
        if (lane == 0) {
            for (int r = 0; r < rule.keep; r++) {
                float best = -INFINITY;
                int at = -1;
                for (int g = 0; g < rule.groups; g++)
                    if (gs[g] != INFINITY && (at < 0 || gs[g] > best)) {
                        best = gs[g];
                        at = g;
                    }
                if (at >= 0) gs[at] = INFINITY;           // kept
            }
        }
        __syncwarp();
        for (int n = lane; n < N; n += 32)
            if (gs[n / size] != INFINITY) c[n] = -INFINITY;
        __syncwarp();
    }
    float picked_sum = 0.0f;
    for (int j = 0; j < top; j++) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int n = lane; n < N; n += 32)
            if (c[n] > best) {                        // ascending n: the first of equals stays
                best = c[n];
                at = n;
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) {
                best = ob;
                at = oa;
            }
        }
        if (at >= N) at = 0;                           // no finite score left (NaN inputs): still a valid index
        if (lane == 0) {
            idx[(size_t)t * top + j] = at;
            weight[(size_t)t * top + j] = s[at];
            c[at] = -INFINITY;
        }
        picked_sum += s[at];
        __syncwarp();
    }
    if (lane == 0) {
        const float div = rule.renorm ? picked_sum + 1e-20f : 1.0f;
        for (int j = 0; j < top; j++) weight[(size_t)t * top + j] = weight[(size_t)t * top + j] / div * rule.scale;
    }
}

template <typename T>
__global__ void __launch_bounds__(32 * MOE_ROUTE_WARPS)
moe_route_kernel(const T* __restrict__ x, const float* __restrict__ router, const float* __restrict__ correction,
                 int* __restrict__ idx, float* __restrict__ weight, int tokens, int D, int N, int top, int vec, MoeRule rule) {
    extern __shared__ float moe_sm[];                 // per warp: scores [N], choice scores [N], runs' scores [groups]
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * MOE_ROUTE_WARPS + warp;
    if (t >= tokens) return;
    float* s = moe_sm + (size_t)warp * (2 * N + rule.groups);
    float* c = s + N;
    const T* xr = x + (size_t)t * D;
    for (int n0 = 0; n0 < N; n0 += 4) {
        const float* w[4];
#pragma unroll
        for (int j = 0; j < 4; j++) w[j] = router + (size_t)min(n0 + j, N - 1) * D;     // past the last output: its sum is dropped
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (vec) {
            // four trips' loads (twenty of them) are issued before the first product needs one: the loop is written out so
            const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int k0 = 4 * lane; k0 < D; k0 += 4 * 128) {
                float4 xv[4], wv[4][4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int k = k0 + 128 * u;
                    const bool ok = k < D;
                    xv[u] = ok ? moe_ld4(xr + k) : zero4;
#pragma unroll
                    for (int j = 0; j < 4; j++) wv[u][j] = ok ? *reinterpret_cast<const float4*>(w[j] + k) : zero4;
                }
#pragma unroll
                for (int u = 0; u < 4; u++)
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        acc[j] = fmaf(xv[u].x, wv[u][j].x, acc[j]);
                        acc[j] = fmaf(xv[u].y, wv[u][j].y, acc[j]);
                        acc[j] = fmaf(xv[u].z, wv[u][j].z, acc[j]);
                        acc[j] = fmaf(xv[u].w, wv[u][j].w, acc[j]);
                    }
            }
        } else {
#pragma unroll 4
            for (int k = lane; k < D; k += 32) {
                const float xv = ld_f(xr + k);
#pragma unroll
                for (int j = 0; j < 4; j++) acc[j] = fmaf(xv, w[j][k], acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float v = warp_sum(acc[j]);
            if (lane == 0 && n0 + j < N) s[n0 + j] = v;
        }
    }
    __syncwarp();
    moe_choose(s, c, c + N, correction, idx, weight, t, N, top, lane, rule);
}

// The same with a block of 1,024 threads per token, for routers small enough that all their partial sums fit in shared
// memory: a warp takes (output, segment of 128 k) items, so the whole router is asked for at once instead of row after
// row (one trip to memory instead of dozens: the warp-per-token form took 75 us whatever the number of tokens); a
// segment's sum is the warp's tree, an output's logit the sum of its segments in ascending order.
#define MOE_ROUTE_WIDE_THREADS 1024
#define MOE_ROUTE_WIDE_ITEMS 8192
template <typename T>
__global__ void __launch_bounds__(MOE_ROUTE_WIDE_THREADS)
moe_route_wide_kernel(const T* __restrict__ x, const float* __restrict__ router, const float* __restrict__ correction,
                      int* __restrict__ idx, float* __restrict__ weight, int D, int N, int top, MoeRule rule) {
    extern __shared__ float moe_sm[];                 // partial sums [N][segs], scores [N], choice scores [N], runs' scores
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x;
    const int segs = (D + 127) / 128;
    float* part = moe_sm;
    float* s = part + (size_t)N * segs;
    float* c = s + N;
    const T* xr = x + (size_t)t * D;
    const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int item = warp; item < N * segs; item += MOE_ROUTE_WIDE_THREADS / 32) {
        const int n = item / segs, k = (item - n * segs) * 128 + 4 * lane;
        const bool ok = k < D;
        const float4 xv = ok ? moe_ld4(xr + k) : zero4;
        const float4 wv = ok ? *reinterpret_cast<const float4*>(router + (size_t)n * D + k) : zero4;
        float a = xv.x * wv.x;
        a = fmaf(xv.y, wv.y, a);
        a = fmaf(xv.z, wv.z, a);
        a = fmaf(xv.w, wv.w, a);
        a = warp_sum(a);
        if (lane == 0) part[item] = a;
    }
    __syncthreads();
    for (int n = threadIdx.x; n < N; n += MOE_ROUTE_WIDE_THREADS) {
        float a = 0.0f;
        for (int g = 0; g < segs; g++) a += part[n * segs + g];
        s[n] = a;
    }
    __syncthreads();
    if (warp > 0) return;
    moe_choose(s, c, c + N, correction, idx, weight, t, N, top, lane, rule);
}

extern "C" int ri_moe_route_rule(const void* x, const float* router, const float* correction, int* idx, float* weight,
                                 int tokens, int D, int N, int top, int mode, int groups, int keep, int gtop, float scale,
                                 int renorm, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(mode == 0 || mode == 1, "moe_route: score rule %d", mode);
    RI_REQUIRE(groups >= 1 && N % groups == 0 && keep >= 1 && keep <= groups && gtop >= 1,
               "moe_route: %d outputs in %d groups of which %d are kept", N, groups, keep);
    RI_REQUIRE(top <= keep * (N / groups), "moe_route: top %d of the %d outputs of the kept groups", top, keep * (N / groups));
    MoeRule rule;
    rule.mode = mode; rule.groups = groups; rule.keep = keep; rule.gtop = gtop; rule.renorm = renorm; rule.scale = scale;
    RI_REQUIRE(tokens > 0 && D > 0 && N > 0 && top > 0 && top <= N, "moe_route: bad sizes (top %d of %d)", top, N);
    RI_REQUIRE(N <= 4096, "moe_route: %d router outputs (up to 4096 are built)", N);
    const size_t smem = (size_t)MOE_ROUTE_WARPS * (2 * N + groups) * sizeof(float);
    const dim3 grid((tokens + MOE_ROUTE_WARPS - 1) / MOE_ROUTE_WARPS);
    // (which form runs depends on the sizes and addresses only, never on the batch)
    const int vec = (D % 4 == 0 && (((uintptr_t)router | (uintptr_t)x) & 15) == 0) ? 1 : 0;
    cudaError_t e = cudaSuccess;
    const long long items = (long long)N * ((D + 127) / 128);
    if (vec && items <= MOE_ROUTE_WIDE_ITEMS && tokens <= 65535 * 32) {
        const size_t sm = (size_t)(items + 2 * N + groups) * sizeof(float);
        if (dtype == RI_DTYPE_F32)
            ri_launch_pdl(moe_route_wide_kernel<float>, dim3(tokens), dim3(MOE_ROUTE_WIDE_THREADS), sm, stream, (const float*)x,
                          router, correction, idx, weight, D, N, top, rule);
        else if (dtype == RI_DTYPE_BF16)
            ri_launch_pdl(moe_route_wide_kernel<bf16>, dim3(tokens), dim3(MOE_ROUTE_WIDE_THREADS), sm, stream, (const bf16*)x,
                          router, correction, idx, weight, D, N, top, rule);
        else RI_FAIL(-1, "moe_route: unknown dtype %d", dtype);
        RI_CHECK_LAUNCH("moe_route");
        return 0;
    }
    if (dtype == RI_DTYPE_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RI_FAIL((int)e, "moe_route: %s", cudaGetErrorString(e));
        ri_launch_pdl(moe_route_kernel<float>, grid, dim3(32 * MOE_ROUTE_WARPS), smem, stream, (const float*)x, router,
                      correction, idx, weight, tokens, D, N, top, vec, rule);
    } else if (dtype == RI_DTYPE_BF16) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_route_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RI_FAIL((int)e, "moe_route: %s", cudaGetErrorString(e));
        ri_launch_pdl(moe_route_kernel<bf16>, grid, dim3(32 * MOE_ROUTE_WARPS), smem, stream, (const bf16*)x, router,
                      correction, idx, weight, tokens, D, N, top, vec, rule);
    } else RI_FAIL(-1, "moe_route: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("moe_route");
    return 0;
}

// ---- the plan ---------------------------------------------------------------------------------------------------------
// meta[0] = number of tiles, meta[1] = number of rows in perm.  tiles [max_tiles][3].
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ idx, int* __restrict__ perm, int* __restrict__ tiles, int* __restrict__ meta,
                int pairs, int E, int max_tiles, int bm) {
    extern __shared__ int plan_sm[];                  // counts [E], offsets [E + 1], cursors [E]
    int* counts = plan_sm;
    int* offsets = counts + E;
    int* cursor = offsets + E + 1;
    pdl_trigger();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = cursor[e] = 0;
    pdl_wait();
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = idx[p];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, n = 0;
        for (int e = 0; e < E; e++) {
            offsets[e] = off;
            for (int r = 0; r < counts[e] && n < max_tiles; r += bm) {
                tiles[3 * n] = e;
                tiles[3 * n + 1] = off + r;
                tiles[3 * n + 2] = min(bm, counts[e] - r);
                n++;
            }
            off += counts[e];
        }
        offsets[E] = off;
        meta[0] = n;
        meta[1] = off;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = idx[p];
        if (e >= 0 && e < E) perm[offsets[e] + atomicAdd(&cursor[e], 1)] = p;
    }
}

// bm: rows per tile, MOE_BM (32) or MOE_BM_WIDE (64: many pairs per expert, bfloat16 with 16-byte rows)
extern "C" int ri_moe_max_tiles(int pairs, int E, int bm) { return (pairs + bm - 1) / bm + E; }

extern "C" int ri_moe_plan(const int* idx, int* perm, int* tiles, int* meta, int pairs, int E, int max_tiles, int bm,
                           cudaStream_t stream) {
    if (pairs == 0) return 0;
    RI_REQUIRE(bm == MOE_BM || bm == MOE_BM_WIDE, "moe_plan: tiles of %d rows are not built", bm);
    RI_REQUIRE(pairs > 0 && E > 0 && max_tiles >= ri_moe_max_tiles(pairs, E, bm), "moe_plan: bad sizes");
    const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
    RI_REQUIRE(smem <= 48 * 1024, "moe_plan: %d experts (up to 4095 are built)", E);
    ri_launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), smem, stream, idx, perm, tiles, meta, pairs, E, max_tiles, bm);
    RI_CHECK_LAUNCH("moe_plan");
    return 0;
}

// ---- grouped products ---------------------------------------------------------------------------------------------------
template <typename TO>
__device__ __forceinline__ void moe_store(TO* p, float v) { st_f(p, v); }

// float32: 128 threads, each 4 rows x 4 columns of the 32 x 64 tile; k ascending, one accumulator per output
template <typename TO>
__global__ void __launch_bounds__(128)
moe_grouped_f32_kernel(const float* __restrict__ a, long long lda, const float* __restrict__ w, TO* __restrict__ y,
                       long long ldy, const int* __restrict__ perm, const int* __restrict__ tiles,
                       const int* __restrict__ meta, int N, int K, int gather_div, int scatter) {
    constexpr int BK = 16;
    __shared__ float As[BK][MOE_BM + 1], Ws[BK][MOE_BN + 1];
    __shared__ int s_in[MOE_BM], s_out[MOE_BM];
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.x >= meta[0]) return;
    const int e = tiles[3 * blockIdx.x], r0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
    const int n0 = blockIdx.y * MOE_BN;
    for (int i = threadIdx.x; i < MOE_BM; i += blockDim.x) {
        const int p = i < rows ? perm[r0 + i] : 0;
        s_in[i] = gather_div > 0 ? p / gather_div : r0 + i;
        s_out[i] = scatter ? p : r0 + i;
    }
    __syncthreads();
    const float* we = w + (size_t)e * N * K;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < MOE_BM * BK; i += blockDim.x) {
            const int r = i / BK, k = i % BK;
            As[k][r] = (r < rows && k0 + k < K) ? a[(size_t)s_in[r] * lda + k0 + k] : 0.0f;
        }
        for (int i = threadIdx.x; i < MOE_BN * BK; i += blockDim.x) {
            const int n = i / BK, k = i % BK;
            Ws[k][n] = (n0 + n < N && k0 + k < K) ? we[(size_t)(n0 + n) * K + k0 + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) wv[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < N) moe_store(y + (size_t)s_out[r] * ldy + n, acc[i][j]);
        }
    }
}

// bfloat16: 4 warps; warp w owns columns 16 w .. 16 w + 15 of the tile and all 32 rows (2 x 2 mma tiles per k16).
// VEC (K a multiple of 8, 16-byte aligned rows): the tiles of A and W come by cp.async through a ring of MOE_STAGES
// stages of 64 k each, so that two stages are on their way while one is multiplied; otherwise element by element.
#define MOE_STAGES 3
#define MOE_BK 64
#define MOE_PITCH (MOE_BK + 8)
template <typename TO, bool VEC>
__global__ void __launch_bounds__(128)
moe_grouped_bf16_kernel(const bf16* __restrict__ a, long long lda, const bf16* __restrict__ w, TO* __restrict__ y,
                        long long ldy, const int* __restrict__ perm, const int* __restrict__ tiles,
                        const int* __restrict__ meta, int N, int K, int gather_div, int scatter) {
    constexpr int ST = VEC ? MOE_STAGES : 1;
    __shared__ __align__(16) bf16 As[ST][MOE_BM][MOE_PITCH], Ws[ST][MOE_BN][MOE_PITCH];
    __shared__ int s_in[MOE_BM], s_out[MOE_BM];
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.x >= meta[0]) return;
    const int e = tiles[3 * blockIdx.x], r0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
    const int n0 = blockIdx.y * MOE_BN;
    for (int i = threadIdx.x; i < MOE_BM; i += blockDim.x) {
        const int p = i < rows ? perm[r0 + i] : 0;
        s_in[i] = gather_div > 0 ? p / gather_div : r0 + i;
        s_out[i] = scatter ? p : r0 + i;
    }
    __syncthreads();
    const bf16* we = w + (size_t)e * N * K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int quad = lane >> 2, qc = lane & 3;
    float acc[2][2][4] = {};
    const bf16 zero = __float2bfloat16_rn(0.0f);
    auto copy_stage = [&](int st, int k0) {        // VEC: 16-byte pieces, zeros past the tile's rows, N and K
#pragma unroll
        for (int pass = 0; pass < 2; pass++) {
            const int i = threadIdx.x + pass * 128;
            const int r = i / 8, kc = (i % 8) * 8;
            const bool ok = r < rows && k0 + kc < K;
            cp_async16(&As[st][r][kc], ok ? a + (size_t)s_in[r] * lda + k0 + kc : a, ok);
        }
#pragma unroll
        for (int pass = 0; pass < 4; pass++) {
            const int i = threadIdx.x + pass * 128;
            const int n = i / 8, kc = (i % 8) * 8;
            const bool ok = n0 + n < N && k0 + kc < K;
            cp_async16(&Ws[st][n][kc], ok ? we + (size_t)(n0 + n) * K + k0 + kc : we, ok);
        }
    };
    auto multiply = [&](int st) {
#pragma unroll
        for (int kk = 0; kk < MOE_BK; kk += 16) {
            unsigned af[2][4], bfr[2][2];
#pragma unroll
            for (int mi = 0; mi < 2; mi++) {
                af[mi][0] = *reinterpret_cast<const unsigned*>(&As[st][mi * 16 + quad][kk + qc * 2]);
                af[mi][1] = *reinterpret_cast<const unsigned*>(&As[st][mi * 16 + quad + 8][kk + qc * 2]);
                af[mi][2] = *reinterpret_cast<const unsigned*>(&As[st][mi * 16 + quad][kk + qc * 2 + 8]);
                af[mi][3] = *reinterpret_cast<const unsigned*>(&As[st][mi * 16 + quad + 8][kk + qc * 2 + 8]);
            }
#pragma unroll
            for (int ni = 0; ni < 2; ni++) {
                bfr[ni][0] = *reinterpret_cast<const unsigned*>(&Ws[st][warp * 16 + ni * 8 + quad][kk + qc * 2]);
                bfr[ni][1] = *reinterpret_cast<const unsigned*>(&Ws[st][warp * 16 + ni * 8 + quad][kk + qc * 2 + 8]);
            }
#pragma unroll
            for (int mi = 0; mi < 2; mi++)
#pragma unroll
                for (int ni = 0; ni < 2; ni++)
                    mma_bf16(acc[mi][ni], af[mi][0], af[mi][1], af[mi][2], af[mi][3], bfr[ni][0], bfr[ni][1]);
        }
    };
    const int nk = (K + MOE_BK - 1) / MOE_BK;
    if (VEC) {
        for (int st = 0; st < MOE_STAGES - 1; st++) {
            if (st < nk) copy_stage(st, st * MOE_BK);
            cp_async_commit();
        }
        for (int it = 0; it < nk; it++) {
            cp_async_wait<MOE_STAGES - 2>();
            __syncthreads();                         // stage `it` has landed for everyone; the stage of it - 1 is free
            const int ahead = it + MOE_STAGES - 1;
            if (ahead < nk) copy_stage(ahead % MOE_STAGES, ahead * MOE_BK);
            cp_async_commit();
            multiply(it % MOE_STAGES);
        }
        cp_async_wait<0>();
    } else {
        for (int it = 0; it < nk; it++) {
            const int k0 = it * MOE_BK;
            for (int i = threadIdx.x; i < MOE_BM * MOE_BK; i += blockDim.x) {
                const int r = i / MOE_BK, k = i % MOE_BK;
                As[0][r][k] = (r < rows && k0 + k < K) ? a[(size_t)s_in[r] * lda + k0 + k] : zero;
            }
            for (int i = threadIdx.x; i < MOE_BN * MOE_BK; i += blockDim.x) {
                const int n = i / MOE_BK, k = i % MOE_BK;
                Ws[0][n][k] = (n0 + n < N && k0 + k < K) ? we[(size_t)(n0 + n) * K + k0 + k] : zero;
            }
            __syncthreads();
            multiply(0);
            __syncthreads();
        }
    }
#pragma unroll
    for (int mi = 0; mi < 2; mi++)
#pragma unroll
        for (int ni = 0; ni < 2; ni++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int r = mi * 16 + quad + (c >> 1) * 8;
                const int n = n0 + warp * 16 + ni * 8 + qc * 2 + (c & 1);
                if (r < rows && n < N) moe_store(y + (size_t)s_out[r] * ldy + n, acc[mi][ni][c]);
            }
}

// Tiles of 64 rows for steps with many pairs per expert (prompts): 2 x 2 warps, each 32 rows x 32 columns (2 x 4 mma
// tiles per k16), fragments by ldmatrix (4 instructions for 8 products), the same ring of cp.async stages in dynamic
// shared memory.  Only with 16-byte rows (K a multiple of 8).
#define MOE_WIDE_SMEM (MOE_STAGES * (MOE_BM_WIDE + MOE_BN) * MOE_PITCH * 2)
template <typename TO>
__global__ void __launch_bounds__(128)
moe_grouped_bf16_wide_kernel(const bf16* __restrict__ a, long long lda, const bf16* __restrict__ w, TO* __restrict__ y,
                             long long ldy, const int* __restrict__ perm, const int* __restrict__ tiles,
                             const int* __restrict__ meta, int N, int K, int gather_div, int scatter) {
    extern __shared__ __align__(16) unsigned char moe_wide_sm[];
    bf16 (*As)[MOE_BM_WIDE][MOE_PITCH] = reinterpret_cast<bf16 (*)[MOE_BM_WIDE][MOE_PITCH]>(moe_wide_sm);
    bf16 (*Ws)[MOE_BN][MOE_PITCH] =
        reinterpret_cast<bf16 (*)[MOE_BN][MOE_PITCH]>(moe_wide_sm + MOE_STAGES * MOE_BM_WIDE * MOE_PITCH * 2);
    __shared__ int s_in[MOE_BM_WIDE], s_out[MOE_BM_WIDE];
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.x >= meta[0]) return;
    const int e = tiles[3 * blockIdx.x], r0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
    const int n0 = blockIdx.y * MOE_BN;
    for (int i = threadIdx.x; i < MOE_BM_WIDE; i += blockDim.x) {
        const int p = i < rows ? perm[r0 + i] : 0;
        s_in[i] = gather_div > 0 ? p / gather_div : r0 + i;
        s_out[i] = scatter ? p : r0 + i;
    }
    __syncthreads();
    const bf16* we = w + (size_t)e * N * K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wm = warp >> 1, wn = warp & 1;
    const int quad = lane >> 2, qc = lane & 3;
    float acc[2][4][4] = {};
    auto copy_stage = [&](int st, int k0) {
#pragma unroll
        for (int pass = 0; pass < 4; pass++) {
            const int i = threadIdx.x + pass * 128;
            const int r = i / 8, kc = (i % 8) * 8;
            const bool ok = r < rows && k0 + kc < K;
            cp_async16(&As[st][r][kc], ok ? a + (size_t)s_in[r] * lda + k0 + kc : a, ok);
        }
#pragma unroll
        for (int pass = 0; pass < 4; pass++) {
            const int i = threadIdx.x + pass * 128;
            const int n = i / 8, kc = (i % 8) * 8;
            const bool ok = n0 + n < N && k0 + kc < K;
            cp_async16(&Ws[st][n][kc], ok ? we + (size_t)(n0 + n) * K + k0 + kc : we, ok);
        }
    };
    const int nk = (K + MOE_BK - 1) / MOE_BK;
    for (int st = 0; st < MOE_STAGES - 1; st++) {
        if (st < nk) copy_stage(st, st * MOE_BK);
        cp_async_commit();
    }
    for (int it = 0; it < nk; it++) {
        cp_async_wait<MOE_STAGES - 2>();
        __syncthreads();
        const int ahead = it + MOE_STAGES - 1;
        if (ahead < nk) copy_stage(ahead % MOE_STAGES, ahead * MOE_BK);
        cp_async_commit();
        const int st = it % MOE_STAGES;
#pragma unroll
        for (int kk = 0; kk < MOE_BK; kk += 16) {
            unsigned af[2][4], bfr[4][2];
#pragma unroll
            for (int mi = 0; mi < 2; mi++)
                ldmatrix_x4(af[mi][0], af[mi][1], af[mi][2], af[mi][3],
                            &As[st][wm * 32 + mi * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
            for (int np = 0; np < 2; np++)          // two n8 tiles per instruction: (b0, b1) of the first, then of the second
                ldmatrix_x4(bfr[2 * np][0], bfr[2 * np][1], bfr[2 * np + 1][0], bfr[2 * np + 1][1],
                            &Ws[st][wn * 32 + np * 16 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
            for (int mi = 0; mi < 2; mi++)
#pragma unroll
                for (int ni = 0; ni < 4; ni++)
                    mma_bf16(acc[mi][ni], af[mi][0], af[mi][1], af[mi][2], af[mi][3], bfr[ni][0], bfr[ni][1]);
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int mi = 0; mi < 2; mi++)
#pragma unroll
        for (int ni = 0; ni < 4; ni++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int r = wm * 32 + mi * 16 + quad + (c >> 1) * 8;
                const int n = n0 + wn * 32 + ni * 8 + qc * 2 + (c & 1);
                if (r < rows && n < N) moe_store(y + (size_t)s_out[r] * ldy + n, acc[mi][ni][c]);
            }
}

// a [rows, lda] and w [E, N, K] in the compute type; y [.., ldy] float32 (out_f32) or the compute type
// bm: the tile height that the plan was made with
extern "C" int ri_moe_grouped_linear(const void* a, long long lda, const void* w, void* y, long long ldy, const int* perm,
                                     const int* tiles, const int* meta, int max_tiles, int bm, int N, int K, int gather_div,
                                     int scatter, int out_f32, int dtype, cudaStream_t stream) {
    if (max_tiles == 0) return 0;
    RI_REQUIRE(bm == MOE_BM || (bm == MOE_BM_WIDE && dtype == RI_DTYPE_BF16), "moe_grouped_linear: tiles of %d rows", bm);
    RI_REQUIRE(max_tiles > 0 && N > 0 && K > 0 && gather_div >= 0, "moe_grouped_linear: bad sizes");
    const dim3 grid(max_tiles, (N + MOE_BN - 1) / MOE_BN);
    RI_REQUIRE(grid.y <= 65535, "moe_grouped_linear: %d outputs are too many for one launch", N);
    if (dtype == RI_DTYPE_F32) {
        RI_REQUIRE(out_f32, "moe_grouped_linear: a float32 product writes float32");
        ri_launch_pdl(moe_grouped_f32_kernel<float>, grid, dim3(128), 0, stream, (const float*)a, lda, (const float*)w,
                      (float*)y, ldy, perm, tiles, meta, N, K, gather_div, scatter);
    } else if (dtype == RI_DTYPE_BF16) {
        const int vec = (K % 8 == 0 && lda % 8 == 0 && (((uintptr_t)a | (uintptr_t)w) & 15) == 0) ? 1 : 0;
        if (bm == MOE_BM_WIDE) {
            RI_REQUIRE(vec, "moe_grouped_linear: tiles of 64 rows need rows of whole 16-byte pieces");
            cudaError_t e1 = cudaFuncSetAttribute(moe_grouped_bf16_wide_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, MOE_WIDE_SMEM);
            cudaError_t e2 = cudaFuncSetAttribute(moe_grouped_bf16_wide_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, MOE_WIDE_SMEM);
            if (e1 != cudaSuccess || e2 != cudaSuccess) RI_FAIL(-1, "moe_grouped_linear: shared memory for the wide tiles");
            if (out_f32)
                ri_launch_pdl(moe_grouped_bf16_wide_kernel<float>, grid, dim3(128), MOE_WIDE_SMEM, stream, (const bf16*)a, lda,
                              (const bf16*)w, (float*)y, ldy, perm, tiles, meta, N, K, gather_div, scatter);
            else
                ri_launch_pdl(moe_grouped_bf16_wide_kernel<bf16>, grid, dim3(128), MOE_WIDE_SMEM, stream, (const bf16*)a, lda,
                              (const bf16*)w, (bf16*)y, ldy, perm, tiles, meta, N, K, gather_div, scatter);
            RI_CHECK_LAUNCH("moe_grouped_linear");
            return 0;
        }
#define MOE_GO(TO, VEC)                                                                                                  \
        ri_launch_pdl(moe_grouped_bf16_kernel<TO, VEC>, grid, dim3(128), 0, stream, (const bf16*)a, lda, (const bf16*)w,    \
                      (TO*)y, ldy, perm, tiles, meta, N, K, gather_div, scatter)
        if (out_f32) {
            if (vec) MOE_GO(float, true); else MOE_GO(float, false);
        } else {
            if (vec) MOE_GO(bf16, true); else MOE_GO(bf16, false);
        }
#undef MOE_GO
    } else RI_FAIL(-1, "moe_grouped_linear: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("moe_grouped_linear");
    return 0;
}

// ---- combination ----------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ pair_out, const int* __restrict__ idx, const float* __restrict__ weight,
                   const T* __restrict__ x, const T* __restrict__ extra, T* __restrict__ y, int D, int top, int E) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < D; d += gridDim.y * blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < top; j++) {
            const int e = idx[(size_t)t * top + j];
            const float v = (e >= E) ? ld_f(x + (size_t)t * D + d) : pair_out[((size_t)t * top + j) * D + d];
            acc = fmaf(weight[(size_t)t * top + j], v, acc);
        }
        if (extra) acc += ld_f(extra + (size_t)t * D + d);
        st_f(y + (size_t)t * D + d, acc);
    }
}

extern "C" int ri_moe_combine(const float* pair_out, const int* idx, const float* weight, const void* x, const void* extra,
                              void* y, int tokens, int D, int top, int E, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    RI_REQUIRE(tokens > 0 && D > 0 && top > 0, "moe_combine: bad sizes");
    const dim3 grid(tokens, tokens >= 512 ? 1 : (D + 255) / 256 > 64 ? 64 : (D + 255) / 256);    // few tokens: a row over several blocks
    if (dtype == RI_DTYPE_F32)
        ri_launch_pdl(moe_combine_kernel<float>, grid, dim3(256), 0, stream, pair_out, idx, weight, (const float*)x,
                      (const float*)extra, (float*)y, D, top, E);
    else if (dtype == RI_DTYPE_BF16)
        ri_launch_pdl(moe_combine_kernel<bf16>, grid, dim3(256), 0, stream, pair_out, idx, weight, (const bf16*)x,
                      (const bf16*)extra, (bf16*)y, D, top, E);
    else RI_FAIL(-1, "moe_combine: unknown dtype %d", dtype);
    RI_CHECK_LAUNCH("moe_combine");
    return 0;
}

extern "C" int ri_moe_route(const void* x, const float* router, const float* correction, int* idx, float* weight,
                            int tokens, int D, int N, int top, int dtype, cudaStream_t stream) {
    return ri_moe_route_rule(x, router, correction, idx, weight, tokens, D, N, top, 0, 1, 1, 1, 1.0f, 1, dtype, stream);
}
