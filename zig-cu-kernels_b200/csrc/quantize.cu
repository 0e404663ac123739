// quantize_fp8_rows / quantize_fp8_tiles for sm_100a: HBM-streaming kernels, 16-byte loads, warp-shuffle amax.
//
// Both kernels work on "octets" (8 consecutive values): one 16-byte load for BF16 input, two for FP32, one 8-byte
// store of E4M3 codes. Algorithmic traffic per value: e bytes read (2 BF16 / 4 FP32) + 1 byte written + s/128 bytes
// of scale (s = 4 FP32 / 1 E8M0).
#include "zck_device.cuh"
#include "zck_host.h"

namespace zck {

template <typename T>
struct Octet;  // 8 values in registers

template <>
struct Octet<__nv_bfloat16> {
    uint4 w;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { w = ld_stream_v4(p); }
    __device__ __forceinline__ void zero() { w = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ float get(int i) const {
        uint32_t word = i < 2 ? w.x : i < 4 ? w.y : i < 6 ? w.z : w.w;
        return (i & 1) ? bf16_hi(word) : bf16_lo(word);
    }
};

template <>
struct Octet<float> {
    uint4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = ld_stream_v4(p);
        b = ld_stream_v4(p + 4);
    }
    __device__ __forceinline__ void zero() { a = b = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ float get(int i) const {
        uint32_t word = i == 0 ? a.x : i == 1 ? a.y : i == 2 ? a.z : i == 3 ? a.w : i == 4 ? b.x : i == 5 ? b.y
                      : i == 6 ? b.z : b.w;
        return __uint_as_float(word);
    }
};

template <typename T>
__device__ __forceinline__ float octet_amax(const Octet<T>& o, float amax) {
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = max_nan(amax, abs_f32(o.get(i)));
    return amax;
}

// Codes of one octet. FP32 scale: x / scale; E8M0 scale: x * 2^(127-b), the same real number, correctly rounded.
template <typename T, bool E8M0>
__device__ __forceinline__ uint2 octet_codes(const Octet<T>& o, const GroupDivider& divide) {
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        if (E8M0) {
            q[i] = __fmul_rn(o.get(i), divide.scale);
            q[i + 1] = __fmul_rn(o.get(i + 1), divide.scale);
        } else {
            const float2 two = divide.pair(o.get(i), o.get(i + 1));
            q[i] = two.x;
            q[i + 1] = two.y;
        }
    }
    return make_uint2(e4m3x4_of(q[0], q[1], q[2], q[3]), e4m3x4_of(q[4], q[5], q[6], q[7]));
}

// ---------------------------------------------------------------------------------------------------------------
// Rows: 8 lanes per scale group, each lane two octets (octet c*8+lane, so every load instruction is contiguous
// over the 8 lanes). Groups are numbered row-major (row * groups_per_row + g). The grid is persistent: a block walks
// group slots with the grid stride and has the loads of its NEXT slot in flight while it reduces, divides and stores
// the current one, so every SM keeps a steady stream of 16-byte loads going.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kRowsThreads = 256;
constexpr int kRowsSlotsPerBlock = kRowsThreads / 8;

template <typename T, bool E8M0, typename Index>
__global__ void __launch_bounds__(kRowsThreads)
quantize_rows_kernel(const T* __restrict__ x, uint64_t x_stride, uint8_t* __restrict__ codes, void* __restrict__ scales,
                     uint64_t scale_stride, uint32_t m, uint32_t groups_per_row) {
    const uint32_t lane = threadIdx.x & 7;
    const Index total = (Index)m * groups_per_row;
    const Index stride = (Index)gridDim.x * kRowsSlotsPerBlock;
    Index slot = (Index)blockIdx.x * kRowsSlotsPerBlock + threadIdx.x / 8;
    // Every thread of a warp runs the same number of iterations (the shuffles need all 32 lanes): the trip count is
    // taken from the first slot of the block, and slots past the end are dead.
    const Index block_first = (Index)blockIdx.x * kRowsSlotsPerBlock;
    Octet<T> next0, next1;
    auto fetch = [&](Index at, Octet<T>& a, Octet<T>& b) {
        if (at < total) {
            const uint32_t row = (uint32_t)(at / groups_per_row), g = (uint32_t)(at % groups_per_row);
            const T* source = x + (uint64_t)row * x_stride + (uint64_t)g * kGroup;
            a.load(source + 8 * lane);
            b.load(source + 8 * (8 + lane));
        } else {
            a.zero();
            b.zero();
        }
    };
    fetch(slot, next0, next1);
    for (Index first = block_first; first < total; first += stride, slot += stride) {
        const Octet<T> o0 = next0, o1 = next1;
        fetch(slot + stride, next0, next1);
        const bool live = slot < total;
        const uint32_t row = live ? (uint32_t)(slot / groups_per_row) : 0, g = live ? (uint32_t)(slot % groups_per_row) : 0;
        float amax = octet_amax(o1, octet_amax(o0, 0.0f));
        amax = max_nan_over_lanes<8>(amax);  // the xor masks 4, 2, 1 stay inside each group of 8 lanes
        float operand;
        if (E8M0) {
            uint32_t byte = scale_e8m0_of(amax);
            operand = e8m0_reciprocal(byte);
            if (live && lane == 0) static_cast<uint8_t*>(scales)[(uint64_t)g * scale_stride + row] = (uint8_t)byte;
        } else {
            operand = scale_f32_of(amax);
            if (live && lane == 0) static_cast<float*>(scales)[(uint64_t)g * scale_stride + row] = operand;
        }
        if (live) {
            // For E8M0 the "divider" only carries the power-of-two factor 2^(127-b) that multiplies every value.
            const GroupDivider divide = GroupDivider::of(operand);
            uint8_t* target = codes + ((uint64_t)row * groups_per_row + g) * kGroup;
            st_global_v2(target + 8 * lane, octet_codes<T, E8M0>(o0, divide));
            st_global_v2(target + 8 * (8 + lane), octet_codes<T, E8M0>(o1, divide));
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Tiles: one block of 256 threads per 128 x 128 tile; thread (r, o) = (t / 16, t % 16) holds octet o of the rows
// pass*16 + r for 8 passes, so the whole tile stays in registers across the single block barrier.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kTilesThreads = 256;

template <typename T, bool E8M0>
__global__ void __launch_bounds__(kTilesThreads)
quantize_tiles_kernel(const T* __restrict__ w, uint64_t w_stride, uint8_t* __restrict__ codes, void* __restrict__ scales,
                      uint64_t scale_stride, uint32_t n, uint32_t k) {
    __shared__ float warp_amax[kTilesThreads / 32];
    const uint32_t tile_col = blockIdx.x, tile_row = blockIdx.y;
    const uint32_t r = threadIdx.x / 16, o = threadIdx.x % 16;
    const uint32_t first_row = tile_row * kGroup;
    const T* source = w + (uint64_t)first_row * w_stride + (uint64_t)tile_col * kGroup + 8 * o;
    Octet<T> held[8];
#pragma unroll
    for (int pass = 0; pass < 8; ++pass) {
        uint32_t row = pass * 16 + r;
        if (first_row + row < n) held[pass].load(source + (uint64_t)row * w_stride);
        else held[pass].zero();
    }
    float amax = 0.0f;
#pragma unroll
    for (int pass = 0; pass < 8; ++pass) amax = octet_amax(held[pass], amax);
    amax = max_nan_over_lanes<32>(amax);
    if ((threadIdx.x & 31) == 0) warp_amax[threadIdx.x / 32] = amax;
    __syncthreads();
    amax = warp_amax[0];
#pragma unroll
    for (int i = 1; i < kTilesThreads / 32; ++i) amax = max_nan(amax, warp_amax[i]);
    float operand;
    if (E8M0) {
        uint32_t byte = scale_e8m0_of(amax);
        operand = e8m0_reciprocal(byte);
        if (threadIdx.x == 0) static_cast<uint8_t*>(scales)[(uint64_t)tile_row * scale_stride + tile_col] = (uint8_t)byte;
    } else {
        operand = scale_f32_of(amax);
        if (threadIdx.x == 0) static_cast<float*>(scales)[(uint64_t)tile_row * scale_stride + tile_col] = operand;
    }
    const GroupDivider divide = GroupDivider::of(operand);
    uint8_t* target = codes + (uint64_t)first_row * k + (uint64_t)tile_col * kGroup + 8 * o;
#pragma unroll
    for (int pass = 0; pass < 8; ++pass) {
        uint32_t row = pass * 16 + r;
        if (first_row + row < n) st_global_v2(target + (uint64_t)row * k, octet_codes<T, E8M0>(held[pass], divide));
    }
}

static int check_quantizer(const void* x, int kind, uint64_t stride, const void* codes, const void* scales,
                           int scale_is_e8m0, uint32_t rows, uint32_t k, const char* name) {
    ZCK_REQUIRE(kind == ZCK_BF16 || kind == ZCK_F32, "%s must be BF16 or FP32", name);
    ZCK_REQUIRE(k % kGroup == 0, "the row length %u of %s is not a multiple of 128", k, name);
    ZCK_REQUIRE(x && codes && scales, "%s, codes and scales must not be NULL", name);
    uint64_t element = kind == ZCK_BF16 ? 2 : 4;
    ZCK_REQUIRE(aligned(x, 16), "%s must start at a multiple of 16 bytes", name);
    ZCK_REQUIRE(rows <= 1 || (stride * element) % 16 == 0, "the row stride of %s must be a multiple of 16 bytes", name);
    ZCK_REQUIRE(rows <= 1 || stride >= k, "the row stride of %s is below the row length", name);
    ZCK_REQUIRE(aligned(codes, 8), "codes must start at a multiple of 8 bytes");
    ZCK_REQUIRE(scale_is_e8m0 || aligned(scales, 4), "FP32 scales must start at a multiple of 4 bytes");
    return ZCK_OK;
}

}  // namespace zck

using namespace zck;

extern "C" int zck_quantize_fp8_rows(const void* x, int x_kind, uint64_t x_stride, void* codes, void* scales,
                                     uint64_t scale_stride, int scale_is_e8m0, uint32_t m, uint32_t k, int device,
                                     void* stream) {
    if (m == 0 || k == 0) return ZCK_OK;
    int code = check_quantizer(x, x_kind, x_stride, codes, scales, scale_is_e8m0, m, k, "x");
    if (code != ZCK_OK) return code;
    DeviceGuard guard(device);
    ZCK_CUDA(guard.error);
    DeviceState* state = device_state(device);
    if (!state) return ZCK_ERR_CUDA;
    uint32_t groups_per_row = k / kGroup;
    uint64_t slots = (uint64_t)m * groups_per_row;
    uint64_t needed = (slots + kRowsSlotsPerBlock - 1) / kRowsSlotsPerBlock;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    dim3 threads(kRowsThreads);
    uint8_t* q = static_cast<uint8_t*>(codes);
    // 32-bit slot arithmetic (one division per slot) whenever the slot count and the grid stride allow it.
    const bool narrow = slots + (uint64_t)state->sm_count * 8 * kRowsSlotsPerBlock < 0xFFFFFFFFull;
    // The grid is persistent, so it holds exactly the blocks that are resident at once (asked of the runtime once per
    // kernel instance).
#define ZCK_ROWS_AS(T, E, I)                                                                                              \
    do {                                                                                                                  \
        static int per_sm = 0;                                                                                            \
        if (per_sm == 0) {                                                                                                \
            int blocks = 0;                                                                                               \
            ZCK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, quantize_rows_kernel<T, E, I>, kRowsThreads, 0)); \
            per_sm = blocks > 0 ? blocks : 1;                                                                             \
        }                                                                                                                 \
        uint64_t resident = (uint64_t)state->sm_count * per_sm;                                                           \
        dim3 grid((unsigned)(needed < resident ? needed : resident));                                                     \
        quantize_rows_kernel<T, E, I><<<grid, threads, 0, s>>>(static_cast<const T*>(x), x_stride, q, scales, scale_stride, m, groups_per_row); \
    } while (0)
#define ZCK_ROWS(T, E)                                   \
    do {                                                 \
        if (narrow) ZCK_ROWS_AS(T, E, uint32_t);         \
        else ZCK_ROWS_AS(T, E, uint64_t);                \
    } while (0)
    if (x_kind == ZCK_BF16) {
        if (scale_is_e8m0) ZCK_ROWS(__nv_bfloat16, true); else ZCK_ROWS(__nv_bfloat16, false);
    } else {
        if (scale_is_e8m0) ZCK_ROWS(float, true); else ZCK_ROWS(float, false);
    }
#undef ZCK_ROWS
#undef ZCK_ROWS_AS
    ZCK_CUDA(cudaGetLastError());
    return ZCK_OK;
}

extern "C" int zck_quantize_fp8_tiles(const void* w, int w_kind, uint64_t w_stride, void* codes, void* scales,
                                      uint64_t scale_stride, int scale_is_e8m0, uint32_t n, uint32_t k, int device,
                                      void* stream) {
    if (n == 0 || k == 0) return ZCK_OK;
    int code = check_quantizer(w, w_kind, w_stride, codes, scales, scale_is_e8m0, n, k, "w");
    if (code != ZCK_OK) return code;
    if (!device_state(device)) return ZCK_ERR_CUDA;
    DeviceGuard guard(device);
    ZCK_CUDA(guard.error);
    uint32_t tile_rows = (n + kGroup - 1) / kGroup, tile_cols = k / kGroup;
    ZCK_REQUIRE(tile_rows <= 65535, "w has too many rows for one launch: %u", n);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    dim3 grid(tile_cols, tile_rows), threads(kTilesThreads);
    uint8_t* q = static_cast<uint8_t*>(codes);
#define ZCK_TILES(T, E) \
    quantize_tiles_kernel<T, E><<<grid, threads, 0, s>>>(static_cast<const T*>(w), w_stride, q, scales, scale_stride, n, k)
    if (w_kind == ZCK_BF16) {
        if (scale_is_e8m0) ZCK_TILES(__nv_bfloat16, true); else ZCK_TILES(__nv_bfloat16, false);
    } else {
        if (scale_is_e8m0) ZCK_TILES(float, true); else ZCK_TILES(float, false);
    }
#undef ZCK_TILES
    ZCK_CUDA(cudaGetLastError());
    return ZCK_OK;
}
