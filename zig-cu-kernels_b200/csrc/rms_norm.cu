// fused_add_rms_norm (and the plain rms_norm it contains) for sm_100a: a one-pass row kernel.
//
// A row lives in registers from its single read to its single write: thread t of the T threads of a row holds the
// 16-byte chunks t, t+T, ... (C of them). h = x + residual is rounded once to the kind of x and stored; the sum of
// squares is reduced by warp shuffles and, for rows wider than a warp, one shared-memory exchange; then
// y = weight (*) kind_of_x(h * rsqrt(mean + eps)).
//
// With block scales (zck_fused_add_rms_norm_quant) the BF16 result is not stored: the 16 (BF16 x) or 32 (FP32 x) lanes
// that hold a group of 128 values agree on its absmax by shuffles and store E4M3 codes and one scale per group, the
// same bits as the row quantizer gives for the BF16 result.
//
// T and C depend on the row width only, never on the row count, so a row gets the same reduction tree in every
// batch (batch invariance). Algorithmic traffic per row of d BF16 values: 2 reads + 2 writes of 2d bytes, + 2d of
// weight (L2 resident).
#include "zck_device.cuh"
#include "zck_host.h"

namespace zck {

struct NormArgs {
    const void* x;
    const void* residual;
    void* residual_out;
    const void* weight;
    const float* fp8_scale;
    void* y;
    void* scales;           // block scales (y_kind kBlockF32 / kBlockE8M0): scales[group * scale_stride + row]
    uint64_t scale_stride;
    uint64_t x_stride, r_stride, ro_stride, y_stride;
    uint32_t rows, width, chunks;  // chunks = width / values per 16-byte chunk of x
    uint32_t threads_per_row;      // T
    int weight_kind, y_kind;
    float eps;
};

template <typename XT>
struct Chunk;  // 16 bytes of x

template <>
struct Chunk<__nv_bfloat16> {
    static constexpr int kValues = 8;
    static __device__ __forceinline__ void unpack(const uint4& w, float (&v)[8]) {
        v[0] = bf16_lo(w.x); v[1] = bf16_hi(w.x); v[2] = bf16_lo(w.y); v[3] = bf16_hi(w.y);
        v[4] = bf16_lo(w.z); v[5] = bf16_hi(w.z); v[6] = bf16_lo(w.w); v[7] = bf16_hi(w.w);
    }
    // Rounds each value to BF16 (nearest even) while packing.
    static __device__ __forceinline__ uint4 pack(const float (&v)[8]) {
        return make_uint4(bf16x2_of(v[0], v[1]), bf16x2_of(v[2], v[3]), bf16x2_of(v[4], v[5]), bf16x2_of(v[6], v[7]));
    }
    static __device__ __forceinline__ float round(float v) { return bf16_round(v); }
};

template <>
struct Chunk<float> {
    static constexpr int kValues = 4;
    static __device__ __forceinline__ void unpack(const uint4& w, float (&v)[4]) {
        v[0] = __uint_as_float(w.x); v[1] = __uint_as_float(w.y); v[2] = __uint_as_float(w.z);
        v[3] = __uint_as_float(w.w);
    }
    static __device__ __forceinline__ uint4 pack(const float (&v)[4]) {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    }
    static __device__ __forceinline__ float round(float v) { return v; }
};

// Weight values of one chunk position as FP32 (and whether they were BF16).
template <int V>
__device__ __forceinline__ void load_weight(const void* weight, int kind, uint32_t first, float (&w)[V]) {
    if ((kind & 3) == ZCK_WEIGHT_BF16) {
        const uint32_t* p = reinterpret_cast<const uint32_t*>(static_cast<const __nv_bfloat16*>(weight) + first);
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
            uint32_t word = __ldg(p + i);
            w[2 * i] = bf16_lo(word);
            w[2 * i + 1] = bf16_hi(word);
        }
    } else {
        const float* p = static_cast<const float*>(weight) + first;
#pragma unroll
        for (int i = 0; i < V; ++i) w[i] = __ldg(p + i);
    }
}

template <int V>
__device__ __forceinline__ void store_y(void* y, int y_kind, uint64_t offset, const float (&v)[V], float fp8_scale) {
    if (y_kind == ZCK_BF16) {
        uint32_t words[V / 2];
#pragma unroll
        for (int i = 0; i < V / 2; ++i) words[i] = bf16x2_of(v[2 * i], v[2 * i + 1]);
        __nv_bfloat16* p = static_cast<__nv_bfloat16*>(y) + offset;
        if (V == 8) st_global_v4(p, make_uint4(words[0], words[1], words[V / 2 - 2], words[V / 2 - 1]));
        else st_global_v2(p, make_uint2(words[0], words[1]));
    } else if (y_kind == ZCK_F32) {
        float* p = static_cast<float*>(y) + offset;
#pragma unroll
        for (int i = 0; i < V / 4; ++i)
            st_global_v4(p + 4 * i, make_uint4(__float_as_uint(v[4 * i]), __float_as_uint(v[4 * i + 1]),
                                               __float_as_uint(v[4 * i + 2]), __float_as_uint(v[4 * i + 3])));
    } else {
        // E4M3 with one caller-given scale: codes of the BF16 result divided by the scale.
        uint32_t words[V / 4];
#pragma unroll
        for (int i = 0; i < V / 4; ++i)
            words[i] = e4m3x4_of(__fdiv_rn(bf16_round(v[4 * i]), fp8_scale), __fdiv_rn(bf16_round(v[4 * i + 1]), fp8_scale),
                                 __fdiv_rn(bf16_round(v[4 * i + 2]), fp8_scale),
                                 __fdiv_rn(bf16_round(v[4 * i + 3]), fp8_scale));
        uint8_t* p = static_cast<uint8_t*>(y) + offset;
        if (V == 8) st_global_v2(p, make_uint2(words[0], words[V / 4 - 1]));
        else *reinterpret_cast<uint32_t*>(p) = words[0];
    }
}

// Internal output kinds next to ZCK_BF16 / ZCK_F32 / ZCK_FP8_E4M3: E4M3 codes with one computed scale per 128 values.
constexpr int kBlockF32 = 16, kBlockE8M0 = 17, kRowF32 = 18;  // kRowF32: one computed FP32 scale per row

// Codes and scale of the V values `v` of one chunk whose group of 128 spans LANES consecutive lanes.
template <int V, int LANES>
__device__ __forceinline__ void store_block_quantized(const NormArgs& a, uint64_t row, uint32_t chunk, float (&v)[V],
                                                      bool live) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        v[i] = bf16_round(v[i]);  // what is quantized is the BF16 result
        amax = max_nan(amax, abs_f32(v[i]));
    }
    // Only the lanes of the group take part (the other half of the warp may hold chunks past the end of the row).
    const uint32_t members = LANES == 32 ? 0xFFFFFFFFu : 0xFFFFu << (threadIdx.x & 16u);
#pragma unroll
    for (int mask = LANES / 2; mask > 0; mask >>= 1) amax = max_nan(amax, __shfl_xor_sync(members, amax, mask));
    const bool e8m0 = a.y_kind == kBlockE8M0;
    const uint32_t group = chunk / LANES;
    float q[V];
    if (e8m0) {
        const uint32_t byte = scale_e8m0_of(amax);
        const float factor = e8m0_reciprocal(byte);
#pragma unroll
        for (int i = 0; i < V; ++i) q[i] = __fmul_rn(v[i], factor);
        if (live && chunk % LANES == 0) static_cast<uint8_t*>(a.scales)[(uint64_t)group * a.scale_stride + row] = (uint8_t)byte;
    } else {
        const float scale = scale_f32_of(amax);
        const GroupDivider divide = GroupDivider::of(scale);
        if (divide.fast) {
#pragma unroll
            for (int i = 0; i < V; i += 2) {
                const float2 two = divide.corrected(v[i], v[i + 1]);
                q[i] = two.x;
                q[i + 1] = two.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) q[i] = __fdiv_rn(v[i], scale);
        }
        if (live && chunk % LANES == 0) static_cast<float*>(a.scales)[(uint64_t)group * a.scale_stride + row] = scale;
    }
    if (!live) return;
    uint8_t* p = static_cast<uint8_t*>(a.y) + row * a.y_stride + (uint64_t)chunk * V;
    if (V == 8) st_global_v2(p, make_uint2(e4m3x4_of(q[0], q[1], q[2], q[3]), e4m3x4_of(q[V - 4], q[V - 3], q[V - 2], q[V - 1])));
    else *reinterpret_cast<uint32_t*>(p) = e4m3x4_of(q[0], q[1], q[2], q[3]);
}

constexpr int kMinBlock = 128;

// Threads per block by instance: rows of up to 128 threads share blocks of 128; C == 8 rows take up to 512 threads
// (BF16, 32768 wide) or 1024 (FP32). The bound lets ptxas keep the whole row in registers.
template <typename XT, int C>
constexpr int max_block() { return C < 8 ? 128 : (sizeof(XT) == 2 ? 512 : 1024); }

template <typename XT, bool ADD, int C>
__global__ void __launch_bounds__(max_block<XT, C>()) rms_norm_kernel(const NormArgs a) {
    constexpr int V = Chunk<XT>::kValues;
    __shared__ float warp_sums[32];
    const uint32_t T = a.threads_per_row;
    const uint32_t rows_per_block = blockDim.x / T;
    const uint32_t t = threadIdx.x % T;
    const uint64_t row = (uint64_t)blockIdx.x * rows_per_block + threadIdx.x / T;
    const bool live = row < a.rows;
    const XT* x = static_cast<const XT*>(a.x) + row * a.x_stride;
    // The row stays packed in the kind of x (4 registers per chunk); h is rounded to that kind anyway.
    uint4 held[C];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        uint32_t chunk = c * T + t;
        held[c] = live && chunk < a.chunks ? ld_stream_v4(x + (uint64_t)chunk * V) : make_uint4(0, 0, 0, 0);
    }
    if (ADD) {
        const XT* r = static_cast<const XT*>(a.residual) + row * a.r_stride;
        XT* out = static_cast<XT*>(a.residual_out) + row * a.ro_stride;
        uint4 other[C];
#pragma unroll
        for (int c = 0; c < C; ++c) {
            uint32_t chunk = c * T + t;
            other[c] = live && chunk < a.chunks ? ld_stream_v4(r + (uint64_t)chunk * V) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int c = 0; c < C; ++c) {
            uint32_t chunk = c * T + t;
            float p[V], q[V];
            Chunk<XT>::unpack(held[c], p);
            Chunk<XT>::unpack(other[c], q);
#pragma unroll
            for (int i = 0; i < V; ++i) p[i] = __fadd_rn(p[i], q[i]);
            held[c] = Chunk<XT>::pack(p);
            if (live && chunk < a.chunks) st_global_v4(out + (uint64_t)chunk * V, held[c]);
        }
    }
    // Sum of squares: two accumulators per thread, then a butterfly over the lanes of the row, then (rows wider
    // than a warp) the per-warp sums of the row added in warp order.
    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        float v[V];
        Chunk<XT>::unpack(held[c], v);
#pragma unroll
        for (int i = 0; i < V; i += 2) {
            s0 = __fmaf_rn(v[i], v[i], s0);
            s1 = __fmaf_rn(v[i + 1], v[i + 1], s1);
        }
    }
    float sum = __fadd_rn(s0, s1);
    const uint32_t lanes = T < 32 ? T : 32;
    for (uint32_t mask = lanes / 2; mask > 0; mask >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xFFFFFFFFu, sum, mask));
    if (T > 32) {
        if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x / 32] = sum;
        __syncthreads();
        const uint32_t warps = T / 32, first = (threadIdx.x / T) * warps;
        sum = warp_sums[first];
        for (uint32_t w = 1; w < warps; ++w) sum = __fadd_rn(sum, warp_sums[first + w]);
    }
    const float scale = rsqrtf(__fadd_rn(__fdiv_rn(sum, (float)a.width), a.eps));
    const float fp8_scale = a.y_kind == ZCK_FP8_E4M3 ? __ldg(a.fp8_scale) : 1.0f;
    const bool zero_centered = (a.weight_kind & ZCK_WEIGHT_ZERO_CENTERED) != 0;
    const int weight = a.weight_kind & 3;
    const bool blocks = a.y_kind == kBlockF32 || a.y_kind == kBlockE8M0, rowwise = a.y_kind == kRowF32;
    if (!live && !blocks && !rowwise) return;  // with computed scales every lane stays for the shuffles and barriers
    // y of chunk position c (zeros past the end of the row).
    auto result_of = [&](int c, float (&y)[V]) {
        const uint32_t chunk = c * T + t;
        Chunk<XT>::unpack(held[c], y);
        if (chunk >= a.chunks) return;
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = __fmul_rn(y[i], scale);
        if (weight != ZCK_WEIGHT_NONE) {
            float w[V];
            load_weight<V>(a.weight, weight, chunk * V, w);
            if (zero_centered) {
#pragma unroll
                for (int i = 0; i < V; ++i) y[i] = __fmul_rn(y[i], __fadd_rn(1.0f, w[i]));
            } else if (weight == ZCK_WEIGHT_BF16) {
                // LlamaRMSNorm: the normalized value is rounded to the kind of x before the weight multiplies it.
#pragma unroll
                for (int i = 0; i < V; ++i) y[i] = __fmul_rn(w[i], Chunk<XT>::round(y[i]));
            } else {
#pragma unroll
                for (int i = 0; i < V; ++i) y[i] = __fmul_rn(w[i], y[i]);
            }
        }
    };
    if (rowwise) {
        // One scale per row: the absmax of the BF16 result over the row (same reduction tree as the sum of squares,
        // NaN kept), then the results once more for the codes.
        float amax = 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            float y[V];
            result_of(c, y);
#pragma unroll
            for (int i = 0; i < V; ++i) amax = max_nan(amax, abs_f32(bf16_round(y[i])));
        }
        for (uint32_t mask = lanes / 2; mask > 0; mask >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, mask));
        if (T > 32) {
            __syncthreads();  // everybody has read the sums
            if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x / 32] = amax;
            __syncthreads();
            const uint32_t warps = T / 32, first = (threadIdx.x / T) * warps;
            amax = warp_sums[first];
            for (uint32_t w = 1; w < warps; ++w) amax = max_nan(amax, warp_sums[first + w]);
        }
        if (!live) return;
        const float row_scale = scale_f32_of(amax);
        if (t == 0) static_cast<float*>(a.scales)[row * a.scale_stride] = row_scale;
        const GroupDivider divide = GroupDivider::of(row_scale);
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const uint32_t chunk = c * T + t;
            if (chunk >= a.chunks) continue;
            float y[V], q[V];
            result_of(c, y);
#pragma unroll
            for (int i = 0; i < V; ++i) q[i] = divide(bf16_round(y[i]));
            uint8_t* p = static_cast<uint8_t*>(a.y) + row * a.y_stride + (uint64_t)chunk * V;
            if (V == 8) st_global_v2(p, make_uint2(e4m3x4_of(q[0], q[1], q[2], q[3]), e4m3x4_of(q[V - 4], q[V - 3], q[V - 2], q[V - 1])));
            else *reinterpret_cast<uint32_t*>(p) = e4m3x4_of(q[0], q[1], q[2], q[3]);
        }
        return;
    }
#pragma unroll
    for (int c = 0; c < C; ++c) {
        uint32_t chunk = c * T + t;
        // Block scales: groups are whole (width % 128 == 0), so the lanes of a group are all in or all out.
        if (chunk >= a.chunks) continue;
        float y[V];
        result_of(c, y);
        if (blocks) store_block_quantized<V, 128 / V>(a, row, chunk, y, live);
        else store_y<V>(a.y, a.y_kind, row * a.y_stride + (uint64_t)chunk * V, y, fp8_scale);
    }
}

// Launch shape from the width alone: C = least of {1,2,4,8} that brings the row to at most 128 threads (8 at most),
// T = threads per row, a power of two below 128 and a multiple of 32 from there on.
static void shape_for(uint32_t chunks, int* c_out, uint32_t* t_out) {
    int c = 1;
    while (c < 8 && (chunks + c - 1) / c > 128) c *= 2;
    uint32_t needed = (chunks + c - 1) / c, t;
    if (needed <= 128) {
        t = 1;
        while (t < needed) t *= 2;
    } else {
        t = (needed + 31) / 32 * 32;
    }
    *c_out = c;
    *t_out = t;
}

template <typename XT, bool ADD>
static cudaError_t launch_norm(const NormArgs& a, int c, cudaStream_t stream) {
    uint32_t T = a.threads_per_row;
    uint32_t block = T >= kMinBlock ? T : kMinBlock;
    uint32_t rows_per_block = block / T;
    uint64_t blocks = ((uint64_t)a.rows + rows_per_block - 1) / rows_per_block;
    dim3 grid((unsigned)blocks), threads(block);
    switch (c) {
        case 1: rms_norm_kernel<XT, ADD, 1><<<grid, threads, 0, stream>>>(a); break;
        case 2: rms_norm_kernel<XT, ADD, 2><<<grid, threads, 0, stream>>>(a); break;
        case 4: rms_norm_kernel<XT, ADD, 4><<<grid, threads, 0, stream>>>(a); break;
        default: rms_norm_kernel<XT, ADD, 8><<<grid, threads, 0, stream>>>(a); break;
    }
    return cudaGetLastError();
}

}  // namespace zck

using namespace zck;

static int norm_entry(const void* x, int x_kind, uint64_t x_stride, const void* residual, uint64_t r_stride,
                      void* residual_out, uint64_t ro_stride, const void* weight, int weight_kind, const float* fp8_scale,
                      void* y, int y_kind, uint64_t y_stride, void* scales, uint64_t scale_stride, uint32_t rows,
                      uint32_t width, float eps, int device, void* stream) {
    if (rows == 0 || width == 0) return ZCK_OK;
    const bool blocks = y_kind == kBlockF32 || y_kind == kBlockE8M0, computed = blocks || y_kind == kRowF32;
    ZCK_REQUIRE(x_kind == ZCK_BF16 || x_kind == ZCK_F32, "x must be BF16 or FP32");
    ZCK_REQUIRE(computed || y_kind == ZCK_BF16 || y_kind == ZCK_F32 || y_kind == ZCK_FP8_E4M3, "y must be BF16, FP32 or E4M3");
    ZCK_REQUIRE(width % 8 == 0, "the row length must be a multiple of 8, got %u", width);
    ZCK_REQUIRE(!blocks || width % kGroup == 0, "block scales need a row length that is a multiple of 128, got %u", width);
    uint32_t x_bytes = x_kind == ZCK_BF16 ? 2 : 4;
    ZCK_REQUIRE((uint64_t)width * x_bytes <= 131072, "rows of %u values are too wide for this kernel", width);
    ZCK_REQUIRE(x && y, "x and y must not be NULL");
    ZCK_REQUIRE(!computed || scales, "scales must not be NULL");
    ZCK_REQUIRE(!computed || y_kind == kBlockE8M0 || aligned(scales, 4), "FP32 scales must start at a multiple of 4 bytes");
    ZCK_REQUIRE((residual == nullptr) == (residual_out == nullptr), "residual and residual_out go together");
    int weight_base = weight_kind & 3;
    ZCK_REQUIRE(weight_base <= ZCK_WEIGHT_F32 && (weight_kind & ~7) == 0, "unknown weight kind %d", weight_kind);
    ZCK_REQUIRE((weight_base == ZCK_WEIGHT_NONE) == (weight == nullptr), "weight and weight_kind disagree");
    ZCK_REQUIRE(!(weight_kind & ZCK_WEIGHT_ZERO_CENTERED) || weight, "zero_centered needs a weight");
    ZCK_REQUIRE((y_kind == ZCK_FP8_E4M3) == (fp8_scale != nullptr), "fp8_scale goes with an E4M3 output only");
    uint32_t y_bytes = y_kind == ZCK_BF16 ? 2 : y_kind == ZCK_F32 ? 4 : 1;
    uint32_t y_align = y_bytes == 1 ? (x_kind == ZCK_BF16 ? 8 : 4) : 16;
    if (y_kind == ZCK_BF16 && x_kind == ZCK_F32) y_align = 8;
    ZCK_REQUIRE(aligned(x, 16) && (rows <= 1 || x_stride * x_bytes % 16 == 0), "x needs 16-byte aligned rows");
    ZCK_REQUIRE(aligned(y, y_align) && (rows <= 1 || y_stride * y_bytes % y_align == 0), "y needs %u-byte aligned rows",
                y_align);
    if (residual) {
        ZCK_REQUIRE(aligned(residual, 16) && (rows <= 1 || r_stride * x_bytes % 16 == 0),
                    "residual needs 16-byte aligned rows");
        ZCK_REQUIRE(aligned(residual_out, 16) && (rows <= 1 || ro_stride * x_bytes % 16 == 0),
                    "residual_out needs 16-byte aligned rows");
    }
    if (weight) ZCK_REQUIRE(aligned(weight, 16), "weight must start at a multiple of 16 bytes");
    if (!device_state(device)) return ZCK_ERR_CUDA;
    DeviceGuard guard(device);
    ZCK_CUDA(guard.error);
    NormArgs a;
    a.x = x; a.residual = residual; a.residual_out = residual_out; a.weight = weight; a.fp8_scale = fp8_scale; a.y = y;
    a.scales = scales; a.scale_stride = scale_stride;
    a.x_stride = x_stride; a.r_stride = r_stride; a.ro_stride = ro_stride; a.y_stride = y_stride;
    a.rows = rows; a.width = width; a.chunks = width * x_bytes / 16;
    a.weight_kind = weight_kind; a.y_kind = y_kind; a.eps = eps;
    int c;
    shape_for(a.chunks, &c, &a.threads_per_row);
    ZCK_REQUIRE(a.threads_per_row <= 1024, "rows of %u values are too wide for this kernel", width);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t error;
    if (x_kind == ZCK_BF16) error = residual ? launch_norm<__nv_bfloat16, true>(a, c, s) : launch_norm<__nv_bfloat16, false>(a, c, s);
    else error = residual ? launch_norm<float, true>(a, c, s) : launch_norm<float, false>(a, c, s);
    if (error != cudaSuccess) return fail(ZCK_ERR_CUDA, "rms_norm launch failed: %s", cudaGetErrorString(error));
    return ZCK_OK;
}

extern "C" int zck_fused_add_rms_norm(const void* x, int x_kind, uint64_t x_stride, const void* residual,
                                      uint64_t r_stride, void* residual_out, uint64_t ro_stride, const void* weight,
                                      int weight_kind, const float* fp8_scale, void* y, int y_kind, uint64_t y_stride,
                                      uint32_t rows, uint32_t width, float eps, int device, void* stream) {
    ZCK_REQUIRE(y_kind == ZCK_BF16 || y_kind == ZCK_F32 || y_kind == ZCK_FP8_E4M3, "y must be BF16, FP32 or E4M3");
    return norm_entry(x, x_kind, x_stride, residual, r_stride, residual_out, ro_stride, weight, weight_kind, fp8_scale, y,
                      y_kind, y_stride, nullptr, 0, rows, width, eps, device, stream);
}

extern "C" int zck_fused_add_rms_norm_quant(const void* x, int x_kind, uint64_t x_stride, const void* residual,
                                            uint64_t r_stride, void* residual_out, uint64_t ro_stride,
                                            const void* weight, int weight_kind, void* codes, uint64_t codes_stride,
                                            void* scales, uint64_t scale_stride, int scale_mode, uint32_t rows,
                                            uint32_t width, float eps, int device, void* stream) {
    ZCK_REQUIRE(scale_mode >= ZCK_SCALES_BLOCK_F32 && scale_mode <= ZCK_SCALES_ROW_F32, "unknown scale mode %d", scale_mode);
    const int kind = scale_mode == ZCK_SCALES_BLOCK_E8M0 ? kBlockE8M0 : scale_mode == ZCK_SCALES_ROW_F32 ? kRowF32 : kBlockF32;
    return norm_entry(x, x_kind, x_stride, residual, r_stride, residual_out, ro_stride, weight, weight_kind, nullptr, codes,
                      kind, codes_stride, scales, scale_stride, rows, width, eps, device, stream);
}
