// Shared-memory ("local") bandwidth and texture-path ("image") bandwidth, the two
// bandwidth rows of the CUDA slot that do not go through plain global loads
// (reference: src/cuda/cuda_kernels/local_bandwidth.cu, image_bandwidth.cu; host
// src/cuda/local_bandwidth.cpp, image_bandwidth.cpp).
#include "../clpk_internal.h"
#include "../clpk_rng.h"

namespace clpk {

constexpr int kLocalReps = 64;          // LMEM_REPS, include/common/common.h:58
constexpr int kImageFetches = 16;       // IMAGE_FETCH_PER_WI, include/common/common.h:61

template <int W> struct Lanes { float v[W]; };

// Every thread stores its W-lane value to its own shared slot, the block meets,
// every thread loads its right-hand neighbour's slot, the block meets again; 64
// rounds.  After them thread t holds what thread (t + 64) % 256 started with, so the
// stored sum is known in closed form.  Bytes counted: 64 rounds x (store + load) x
// 4W bytes per thread, the reference's accounting.
template <int W>
__global__ void __launch_bounds__(256) local_bandwidth_kernel(float *__restrict__ out)
{
    __shared__ __align__(16) Lanes<W> slot[256];
    const uint32_t t = threadIdx.x, gid = blockIdx.x * 256u + t, right = (t + 1u) & 255u;
    Lanes<W> mine;
#pragma unroll
    for (int l = 0; l < W; l++)
        mine.v[l] = (float)(gid + (uint32_t)l);
#pragma unroll 1
    for (int r = 0; r < kLocalReps; r++) {
        slot[t] = mine;
        __syncthreads();
        mine = slot[right];
        __syncthreads();
    }
    float s = mine.v[0];
#pragma unroll
    for (int l = 1; l < W; l++)
        s = __fadd_rn(s, mine.v[l]);
    out[gid] = s;
}

// Texel (x, y), channel ch = uniform[0,1) number 4*(y*width + x) + ch of the seed.
__global__ void image_fill_kernel(float4 *__restrict__ texels, uint64_t n_texels, uint64_t seed)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_texels; i += stride)
        texels[i] = make_float4(clpk_uniform01(seed, 4 * i), clpk_uniform01(seed, 4 * i + 1),
                                clpk_uniform01(seed, 4 * i + 2), clpk_uniform01(seed, 4 * i + 3));
}

// 16 point-sampled float4 fetches per thread, fetch i at texel (gid + i * threads) mod
// (width * height); channel-wise sums, then x + y + z + w.  With threads * 16 =
// width * height every texel is read exactly once per launch.
template <bool POW2>
__global__ void __launch_bounds__(256) image_bandwidth_kernel(cudaTextureObject_t tex, float *__restrict__ out,
                                                              uint32_t width, uint32_t total, uint32_t shift)
{
    // the host checks threads * 16 <= 2^31 - 1, so 32-bit unsigned texel numbers cannot wrap
    const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t threads = gridDim.x * blockDim.x;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < kImageFetches; i++) {
        uint32_t texel = gid + (uint32_t)i * threads;
        if (texel >= total)
            texel %= total;
        const uint32_t x = POW2 ? (texel & (width - 1u)) : texel % width;
        const uint32_t y = POW2 ? (texel >> shift) : texel / width;
        const float4 v = tex2D<float4>(tex, (int)x, (int)y);
        sum.x = __fadd_rn(sum.x, v.x);
        sum.y = __fadd_rn(sum.y, v.y);
        sum.z = __fadd_rn(sum.z, v.z);
        sum.w = __fadd_rn(sum.w, v.w);
    }
    out[gid] = __fadd_rn(__fadd_rn(__fadd_rn(sum.x, sum.y), sum.z), sum.w);
}

// The same 16 fetches per thread, laid out for the texture cache and the block-linear array
// instead of in the reference's order: a warp reads a 4 x 8 patch of texels, the eight warps of a
// block an 8 x 32 one, and the block's 16 fetches are 16 neighbouring patches (patch number
// block * 16 + i, patches numbered along x, modulo their count).  Every texel is still read
// exactly once when threads * 16 = width * height.  Measured on a B200 with the 4096 x 4096
// float4 image: 6.2 TB/s against 4.5 for the order above, in which a block's fetches lie
// 256 rows apart.
constexpr int kPatchW = 4, kPatchH = 8, kBlockPatchesX = 2, kBlockPatchesY = 4;
constexpr int kTileW = kPatchW * kBlockPatchesX, kTileH = kPatchH * kBlockPatchesY;      // 8 x 32 texels

__global__ void __launch_bounds__(256) image_bandwidth_tiled_kernel(cudaTextureObject_t tex, float *__restrict__ out,
                                                                    uint32_t tiles_x, uint32_t n_tiles)
{
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t dx = (warp % kBlockPatchesX) * kPatchW + lane % kPatchW;
    const uint32_t dy = (warp / kBlockPatchesX) * kPatchH + lane / kPatchW;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < kImageFetches; i++) {
        uint32_t tile = blockIdx.x * (uint32_t)kImageFetches + (uint32_t)i;
        if (tile >= n_tiles)
            tile %= n_tiles;
        const uint32_t tx = tile % tiles_x, ty = tile / tiles_x;
        const float4 v = tex2D<float4>(tex, (int)(tx * kTileW + dx), (int)(ty * kTileH + dy));
        sum.x = __fadd_rn(sum.x, v.x);
        sum.y = __fadd_rn(sum.y, v.y);
        sum.z = __fadd_rn(sum.z, v.z);
        sum.w = __fadd_rn(sum.w, v.w);
    }
    out[blockIdx.x * 256u + threadIdx.x] = __fadd_rn(__fadd_rn(__fadd_rn(sum.x, sum.y), sum.z), sum.w);
}

struct Image {
    cudaArray_t array = nullptr;
    cudaTextureObject_t tex = 0;
    uint32_t width = 0, height = 0;
};

} // namespace clpk

using namespace clpk;

extern "C" {

int clpk_local_bandwidth(int width, float *d_out, uint32_t grid, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(width == 1 || width == 2 || width == 4, "width must be 1, 2 or 4 (got %d)", width);
    CLPK_REQUIRE(d_out && grid > 0, "bad arguments");
    cudaStream_t s = as_stream(stream);
    if (width == 1)
        local_bandwidth_kernel<1><<<grid, 256, 0, s>>>(d_out);
    else if (width == 2)
        local_bandwidth_kernel<2><<<grid, 256, 0, s>>>(d_out);
    else
        local_bandwidth_kernel<4><<<grid, 256, 0, s>>>(d_out);
    CLPK_LAUNCH_CHECK("local_bandwidth");
    return CLPK_OK;
}

int clpk_image_create(void **image, uint32_t width, uint32_t height, uint64_t seed, void *stream)
{
    int rc = require_sm100();
    if (rc != CLPK_OK)
        return rc;
    CLPK_REQUIRE(image, "image is NULL");
    *image = nullptr;
    CLPK_REQUIRE(width > 0 && height > 0 && width <= 65536 && height <= 65536 &&
                     (uint64_t)width * height <= 0x7FFFFFFFull,
                 "image size %u x %u out of range", width, height);
    cudaStream_t s = as_stream(stream);
    const uint64_t n = (uint64_t)width * height;
    float4 *linear = nullptr;
    CLPK_CUDA(cudaMalloc(&linear, n * sizeof(float4)));
    Image *img = new Image;
    img->width = width;
    img->height = height;
    auto fail = [&](cudaError_t e, const char *what) {
        cudaFree(linear);
        if (img->tex)
            cudaDestroyTextureObject(img->tex);
        if (img->array)
            cudaFreeArray(img->array);
        delete img;
        return cuda_fail(e, what);
    };
    const cudaChannelFormatDesc fmt = cudaCreateChannelDesc<float4>();
    cudaError_t e = cudaMallocArray(&img->array, &fmt, width, height);
    if (e != cudaSuccess)
        return fail(e, "cudaMallocArray");
    const int sms = num_sms();
    image_fill_kernel<<<(sms > 0 ? sms : 128) * 8, 256, 0, s>>>(linear, n, seed);
    e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(e, "launch image_fill");
    e = cudaMemcpy2DToArrayAsync(img->array, 0, 0, linear, (size_t)width * sizeof(float4),
                                 (size_t)width * sizeof(float4), height, cudaMemcpyDeviceToDevice, s);
    if (e != cudaSuccess)
        return fail(e, "cudaMemcpy2DToArrayAsync");
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess)
        return fail(e, "cudaStreamSynchronize");
    cudaResourceDesc rd = {};
    rd.resType = cudaResourceTypeArray;
    rd.res.array.array = img->array;
    cudaTextureDesc td = {};
    td.addressMode[0] = td.addressMode[1] = cudaAddressModeClamp;
    td.filterMode = cudaFilterModePoint;
    td.readMode = cudaReadModeElementType;
    td.normalizedCoords = 0;
    e = cudaCreateTextureObject(&img->tex, &rd, &td, nullptr);
    if (e != cudaSuccess)
        return fail(e, "cudaCreateTextureObject");
    cudaFree(linear);
    *image = img;
    return CLPK_OK;
}

int clpk_image_bandwidth(void *image, float *d_out, uint32_t grid, void *stream)
{
    CLPK_REQUIRE(image && d_out && grid > 0, "bad arguments");
    const Image *img = static_cast<const Image *>(image);
    CLPK_REQUIRE((uint64_t)grid * 256 <= 0x7FFFFFFFull / kImageFetches, "grid %u too large", grid);
    const uint32_t total = img->width * img->height;
    if ((img->width & (img->width - 1u)) == 0) {
        uint32_t shift = 0;
        while ((1u << shift) < img->width)
            shift++;
        image_bandwidth_kernel<true><<<grid, 256, 0, as_stream(stream)>>>(img->tex, d_out, img->width, total, shift);
    } else {
        image_bandwidth_kernel<false><<<grid, 256, 0, as_stream(stream)>>>(img->tex, d_out, img->width, total, 0);
    }
    CLPK_LAUNCH_CHECK("image_bandwidth");
    return CLPK_OK;
}

int clpk_image_bandwidth_tiled(void *image, float *d_out, uint32_t grid, void *stream)
{
    CLPK_REQUIRE(image && d_out && grid > 0, "bad arguments");
    const Image *img = static_cast<const Image *>(image);
    CLPK_REQUIRE(img->width % kTileW == 0 && img->height % kTileH == 0,
                 "the tiled order needs a width that is a multiple of %d and a height that is a multiple of %d (got %u x %u)",
                 kTileW, kTileH, img->width, img->height);
    CLPK_REQUIRE((uint64_t)grid * kImageFetches <= 0xFFFFFFFFull, "grid %u too large", grid);
    const uint32_t tiles_x = img->width / kTileW, n_tiles = tiles_x * (img->height / kTileH);
    image_bandwidth_tiled_kernel<<<grid, 256, 0, as_stream(stream)>>>(img->tex, d_out, tiles_x, n_tiles);
    CLPK_LAUNCH_CHECK("image_bandwidth_tiled");
    return CLPK_OK;
}

int clpk_image_destroy(void *image)
{
    if (!image)
        return CLPK_OK;
    Image *img = static_cast<Image *>(image);
    cudaError_t e1 = cudaDestroyTextureObject(img->tex);
    cudaError_t e2 = cudaFreeArray(img->array);
    delete img;
    if (e1 != cudaSuccess)
        return cuda_fail(e1, "cudaDestroyTextureObject");
    if (e2 != cudaSuccess)
        return cuda_fail(e2, "cudaFreeArray");
    return CLPK_OK;
}

} // extern "C"
