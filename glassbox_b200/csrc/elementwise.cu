// Embedding gather, RMSNorm, rotary encoding fused with the cache write, SwiGLU activation,
// page copy. All statistics and the residual stream are float32; only the stored activations
// (and the cache) take the compute dtype.
#include "common.cuh"

// ----------------------------------------------------------------------------------------------
// Embedding: x[i, :] = table[tokens[i], :]   (crates/glassbox-core/src/model.rs:228-231)
// ----------------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ x,
                             int n, int d, int vocab, int* __restrict__ status) {
    int row = blockIdx.x;
    if (row >= n) return;
    int tok = tokens[row];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < d; j += blockDim.x) x[(size_t)row * d + j] = 0.f;
        return;
    }
    const TW* src = table + (size_t)tok * d;
    for (int j = threadIdx.x; j < d; j += blockDim.x) x[(size_t)row * d + j] = gb_to_float(src[j]);
}

GB_EXPORT int gb_embed(const void* table, int table_dtype, const int* tokens, float* x, int n, int d, int vocab,
                       int* status, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0 && vocab > 0, "gb_embed: bad sizes n=%d d=%d vocab=%d", n, d, vocab);
    if (n == 0) return 0;
    int threads = d >= 256 ? 256 : 128;
    if (table_dtype == GB_F32)
        embed_kernel<float><<<n, threads, 0, stream>>>((const float*)table, tokens, x, n, d, vocab, status);
    else if (table_dtype == GB_BF16)
        embed_kernel<__nv_bfloat16><<<n, threads, 0, stream>>>((const __nv_bfloat16*)table, tokens, x, n, d, vocab,
                                                                status);
    else
        GB_REQUIRE(false, "gb_embed: unsupported table dtype %d", table_dtype);
    return gb_check_launch("gb_embed");
}

// ----------------------------------------------------------------------------------------------
// RMSNorm: out_j = w_j * (x_j * rsqrt(mean(x^2) + eps))   (crates/glassbox-core/src/model.rs:94-100)
// `rows` (optional) gathers input rows, used for the final norm on the wanted rows only.
// ----------------------------------------------------------------------------------------------
template <typename TO, int THREADS>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                               const float* __restrict__ gain, TO* __restrict__ out, int n, int d, float eps) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    int r = blockIdx.x;
    if (r >= n) return;
    const float* src = x + (size_t)(rows ? rows[r] : r) * d;
    TO* dst = out + (size_t)r * d;
    __shared__ float partial[THREADS / 32];
    __shared__ float total;
    // A row of up to THREADS * 4 * VMAX values whose pieces of four are aligned is read once, every load in
    // flight at the same time, and normalised from registers (instructions issue in order: a loop that uses each
    // value as it arrives pays the memory latency once per round). Longer or unaligned rows take two passes.
    constexpr int VMAX = 4;
    const bool quick = d % 4 == 0 && d <= THREADS * 4 * VMAX && ((uintptr_t)src & 15) == 0 && ((uintptr_t)gain & 15) == 0;
    float4 v[VMAX];
    float ss = 0.f;
    if (quick) {
#pragma unroll
        for (int i = 0; i < VMAX; ++i) {
            const int j = (i * THREADS + threadIdx.x) * 4;
            v[i] = j < d ? *reinterpret_cast<const float4*>(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < VMAX; ++i) {
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    } else {
        for (int j = threadIdx.x; j < d; j += THREADS) {
            float t = src[j];
            ss = fmaf(t, t, ss);
        }
    }
    ss = gb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < THREADS / 32; ++w) t += partial[w];
        total = 1.0f / sqrtf(t / (float)d + eps);
    }
    __syncthreads();
    float s = total;
    if (quick) {
#pragma unroll
        for (int i = 0; i < VMAX; ++i) {
            const int j = (i * THREADS + threadIdx.x) * 4;
            if (j < d) {
                const float4 g = *reinterpret_cast<const float4*>(gain + j);
                const float y0 = g.x * (v[i].x * s), y1 = g.y * (v[i].y * s), y2 = g.z * (v[i].z * s), y3 = g.w * (v[i].w * s);
                if constexpr (sizeof(TO) == 2) {
                    if (((uintptr_t)(dst + j) & 7) == 0) {
                        __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
                        uint2 w;
                        w.x = *reinterpret_cast<uint32_t*>(&lo);
                        w.y = *reinterpret_cast<uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(dst + j) = w;
                        continue;
                    }
                }
                dst[j] = gb_from_float<TO>(y0);
                dst[j + 1] = gb_from_float<TO>(y1);
                dst[j + 2] = gb_from_float<TO>(y2);
                dst[j + 3] = gb_from_float<TO>(y3);
            }
        }
    } else {
        for (int j = threadIdx.x; j < d; j += THREADS) dst[j] = gb_from_float<TO>(gain[j] * (src[j] * s));
    }
}

GB_EXPORT int gb_rmsnorm(const float* x, const int* rows, const float* gain, void* out, int out_dtype, int n, int d,
                         float eps, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0, "gb_rmsnorm: bad sizes n=%d d=%d", n, d);
    if (n == 0) return 0;
    if (out_dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, rmsnorm_kernel<float, 128>, dim3(n), dim3(128), 0, stream, x, rows, gain, (float*)out, n, d, eps);
    else if (out_dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, rmsnorm_kernel<__nv_bfloat16, 128>, dim3(n), dim3(128), 0, stream, x, rows, gain, (__nv_bfloat16*)out, n, d,
                  eps);
    else
        GB_REQUIRE(false, "gb_rmsnorm: unsupported output dtype %d", out_dtype);
    return gb_check_launch("gb_rmsnorm");
}

// ----------------------------------------------------------------------------------------------
// Rotary encoding of q and k at each row's own position, fused with the cache write.
// Pair (i, i + rot/2): x_i' = x_i c - x_{i+rot/2} s ; x_{i+rot/2}' = x_{i+rot/2} c + x_i s
// (crates/glassbox-core/src/model.rs:102-115, 266-276). cos/sin come from a float32 table
// [max_position, rot/2] of (cos, sin) built on the host. K is stored after rotation.
// Cache layout per cache layer: [page, kv_head, page_size, head_dim]; slot = page*page_size + offset.
// With table == nullptr nothing is rotated (a mixer without position encoding).
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const float2* __restrict__ table,
                                     const int* __restrict__ positions, const int* __restrict__ slots,
                                     T* __restrict__ kcache, T* __restrict__ vcache, int n, int nh, int nkv, int hd,
                                     int rot, int max_pos, int page_size, long long num_slots, int write_kv,
                                     int* __restrict__ status) {
    // (launched without programmatic serialisation: letting the attention kernel that follows start early
    // cost 9 % of a decode step at batch 64 with SmolLM2-1.7B shapes and gained 1 % of a prefill step)
    int row = blockIdx.x;
    if (row >= n) return;
    const int qd = nh * hd, kvd = nkv * hd;
    T* base = qkv + (size_t)row * (qd + 2 * kvd);
    int pos = positions[row];
    if (pos < 0) return;  // a padding row of a fixed-shape batch: nothing to rotate, nothing to store
    bool rotate = table != nullptr;
    if (rotate && (pos < 0 || pos >= max_pos)) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        rotate = false;
    }
    const int half = rot / 2;
    const float2* cs = rotate ? table + (size_t)pos * half : nullptr;
    long long slot = slots[row];
    bool store = write_kv != 0;
    if (store && (slot < 0 || slot >= num_slots)) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_SLOT);
        store = false;
    }
    const long long page = slot / page_size;
    const int off = (int)(slot % page_size);

    // q heads: rotate in place.
    if (rotate) {
        for (int idx = threadIdx.x; idx < nh * half; idx += blockDim.x) {
            int h = idx / half, i = idx % half;
            float2 c = cs[i];
            T* p = base + h * hd;
            float x0 = gb_to_float(p[i]), x1 = gb_to_float(p[i + half]);
            p[i] = gb_from_float<T>(x0 * c.x - x1 * c.y);
            p[i + half] = gb_from_float<T>(x1 * c.x + x0 * c.y);
        }
    }
    // k heads: rotate, store to the cache (and back in place, so that callers may read it).
    for (int idx = threadIdx.x; idx < nkv * (hd / 2); idx += blockDim.x) {
        int h = idx / (hd / 2), i = idx % (hd / 2);
        T* p = base + qd + h * hd;
        // Channels below `rot` come in pairs (i, i+half); channels at or above `rot` pass through.
        // Work on two channels per thread: a = 2*i' mapping chosen so every channel is visited once.
        int c0, c1;
        float y0, y1;
        if (i < half) {
            c0 = i;
            c1 = i + half;
            float x0 = gb_to_float(p[c0]), x1 = gb_to_float(p[c1]);
            if (rotate) {
                float2 c = cs[i];
                y0 = x0 * c.x - x1 * c.y;
                y1 = x1 * c.x + x0 * c.y;
            } else {
                y0 = x0;
                y1 = x1;
            }
        } else {
            c0 = rot + 2 * (i - half);
            c1 = c0 + 1;
            y0 = gb_to_float(p[c0]);
            y1 = gb_to_float(p[c1]);
        }
        T t0 = gb_from_float<T>(y0), t1 = gb_from_float<T>(y1);
        p[c0] = t0;
        p[c1] = t1;
        if (store) {
            T* dst = kcache + (((size_t)page * nkv + h) * page_size + off) * hd;
            dst[c0] = t0;
            dst[c1] = t1;
        }
    }
    if (store) {
        const T* v = base + qd + kvd;
        for (int idx = threadIdx.x; idx < kvd; idx += blockDim.x) {
            int h = idx / hd, i = idx % hd;
            vcache[(((size_t)page * nkv + h) * page_size + off) * hd + i] = v[idx];
        }
    }
}

GB_EXPORT int gb_rope_kv_write(void* qkv, int dtype, const float* cos_sin, const int* positions, const int* slots,
                               void* kcache, void* vcache, int n, int nh, int nkv, int hd, int rot, int max_pos,
                               int page_size, long long num_pages, int write_kv, int* status, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && nh > 0 && nkv > 0 && hd > 0 && hd % 2 == 0, "gb_rope_kv_write: bad sizes");
    GB_REQUIRE(rot >= 0 && rot <= hd && rot % 2 == 0, "gb_rope_kv_write: rotary dim %d must be even and <= head dim %d",
               rot, hd);
    GB_REQUIRE(page_size > 0, "gb_rope_kv_write: page size must be positive");
    if (n == 0) return 0;
    long long num_slots = num_pages * page_size;
    const float2* table = rot > 0 ? (const float2*)cos_sin : nullptr;
    if (dtype == GB_F32)
        gb_launch(0, rope_kv_write_kernel<float>, dim3(n), dim3(128), 0, stream, (float*)qkv, table, positions, slots,
                  (float*)kcache, (float*)vcache, n, nh, nkv, hd, rot, max_pos, page_size, num_slots, write_kv, status);
    else if (dtype == GB_BF16)
        gb_launch(0, rope_kv_write_kernel<__nv_bfloat16>, dim3(n), dim3(128), 0, stream, (__nv_bfloat16*)qkv, table, positions,
                  slots, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, n, nh, nkv, hd, rot, max_pos, page_size, num_slots,
                  write_kv, status);
    else
        GB_REQUIRE(false, "gb_rope_kv_write: unsupported dtype %d", dtype);
    return gb_check_launch("gb_rope_kv_write");
}

// ----------------------------------------------------------------------------------------------
// SwiGLU activation: act = g / (1 + exp(-g)) * u, gate in columns [0, I), up in [I, 2I)
// (crates/glassbox-core/src/model.rs:336-340). Computed in float32.
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, long long n, int inter) {
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long total = n * inter;
    for (; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        long long r = idx / inter;
        int j = (int)(idx % inter);
        float g = gb_to_float(gu[r * 2 * inter + j]);
        float u = gb_to_float(gu[r * 2 * inter + inter + j]);
        act[idx] = gb_from_float<T>(g / (1.0f + expf(-g)) * u);
    }
}

GB_EXPORT int gb_swiglu(const void* gate_up, void* act, int dtype, int n, int inter, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && inter > 0, "gb_swiglu: bad sizes n=%d I=%d", n, inter);
    if (n == 0) return 0;
    long long total = (long long)n * inter;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == GB_F32)
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)act, n, inter);
    else if (dtype == GB_BF16)
        swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)act,
                                                                  n, inter);
    else
        GB_REQUIRE(false, "gb_swiglu: unsupported dtype %d", dtype);
    return gb_check_launch("gb_swiglu");
}

// ----------------------------------------------------------------------------------------------
// Page copy for copy-on-write: for each pair, copy one page of K and V in every cache layer of a
// group (crates/glassbox-core/src/kv.rs:189-196). Layers are `layer_stride` elements apart.
// ----------------------------------------------------------------------------------------------
__global__ void copy_pages_kernel(uint4* __restrict__ k, uint4* __restrict__ v, const int* __restrict__ pairs,
                                  int n_pairs, long long page_vec, long long layer_vec, int layers) {
    int pair = blockIdx.x, layer = blockIdx.y;
    if (pair >= n_pairs || layer >= layers) return;
    long long src = pairs[2 * pair], dst = pairs[2 * pair + 1];
    uint4* ks = k + layer * layer_vec + src * page_vec;
    uint4* kd = k + layer * layer_vec + dst * page_vec;
    uint4* vs = v + layer * layer_vec + src * page_vec;
    uint4* vd = v + layer * layer_vec + dst * page_vec;
    for (long long i = threadIdx.x; i < page_vec; i += blockDim.x) {
        kd[i] = ks[i];
        vd[i] = vs[i];
    }
}

GB_EXPORT int gb_copy_pages(void* kcache, void* vcache, const int* pairs, int n_pairs, long long page_bytes,
                            long long layer_bytes, int layers, cudaStream_t stream) {
    GB_REQUIRE(page_bytes % 16 == 0 && layer_bytes % 16 == 0, "gb_copy_pages: page bytes must be a multiple of 16");
    if (n_pairs == 0 || layers == 0) return 0;
    dim3 grid(n_pairs, layers);
    copy_pages_kernel<<<grid, 256, 0, stream>>>((uint4*)kcache, (uint4*)vcache, pairs, n_pairs, page_bytes / 16,
                                                layer_bytes / 16, layers);
    return gb_check_launch("gb_copy_pages");
}
