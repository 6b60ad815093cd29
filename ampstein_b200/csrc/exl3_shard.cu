// Tensor-parallel shards of an EXL3 linear cut on the device, in one launch per shard, straight into
// their final buffer (which may be another GPU's memory when peer access is enabled: plain 16-byte
// stores, no staging copy).
//
// Replaces the narrow + torch.cat + contiguous + .cuda(dev) chains of the reference's load path
// (sub_columns / cols / rows, src/ucode/ampstein/models.uc:440-562). A column shard is the
// concatenation of 128-aligned column ranges: in the trellis (k/16, n/16, 16K) a range is, per tile
// row, one contiguous run of (length / 16) tiles of 32K bytes; svh is sliced the same way. A row
// shard is a leading-dimension slice (two contiguous copies). Byte moves only: bit-exact.
#include "host_common.h"
#include "../../include/ampstein_b200.h"
#include <cstdint>

namespace amp {

constexpr int SHARD_MAX_RANGES = 16;

struct ShardCols
{
    const unsigned char* trellis; unsigned char* out;
    const unsigned char* svh; unsigned char* out_svh;
    long tile_row_bytes_in, tile_row_bytes_out;         // n / 16 * 32K and nsub / 16 * 32K
    int tile_bytes, nranges, tile_rows;
    int start[SHARD_MAX_RANGES], length[SHARD_MAX_RANGES], out_start[SHARD_MAX_RANGES];      // columns
};

// blockIdx.y = range, blockIdx.x walks the tile rows; a block copies the range's run of one tile row
// (16 bytes per thread and step); the block of tile row 0 also copies the range's svh values
__global__ __launch_bounds__(256)
void shard_cols_kernel(const ShardCols P)
{
    const int r = blockIdx.y;
    const size_t run = (size_t) (P.length[r] >> 4) * P.tile_bytes;                       // bytes per tile row, a multiple of 256
    const size_t src0 = (size_t) (P.start[r] >> 4) * P.tile_bytes, dst0 = (size_t) (P.out_start[r] >> 4) * P.tile_bytes;
    for (int kt = blockIdx.x; kt < P.tile_rows; kt += gridDim.x)
    {
        const uint4* src = reinterpret_cast<const uint4*>(P.trellis + (size_t) kt * P.tile_row_bytes_in + src0);
        uint4* dst = reinterpret_cast<uint4*>(P.out + (size_t) kt * P.tile_row_bytes_out + dst0);
        for (size_t i = threadIdx.x; i < (run >> 4); i += blockDim.x) dst[i] = __ldcs(src + i);
    }
    if (blockIdx.x == 0 && P.svh)
    {
        const uint4* src = reinterpret_cast<const uint4*>(P.svh + (size_t) P.start[r] * 2);
        uint4* dst = reinterpret_cast<uint4*>(P.out_svh + (size_t) P.out_start[r] * 2);
        for (int i = threadIdx.x; i < (P.length[r] >> 3); i += blockDim.x) dst[i] = src[i];
    }
}

}  // namespace amp

using namespace amp;

AMP_API int amp_exl3_shard_cols(const void* trellis, const void* svh, void* out_trellis, void* out_svh, int k, int n, int K,
                                const int* ranges, int nranges, cudaStream_t stream)
{
    AMP_REQUIRE(trellis && out_trellis && ranges, "exl3_shard_cols: null pointer");
    AMP_REQUIRE((svh == nullptr) == (out_svh == nullptr), "exl3_shard_cols: give svh and its destination, or neither");
    AMP_REQUIRE(k > 0 && n > 0 && k % 16 == 0 && n % 16 == 0 && ((K >= 1 && K <= 8) || (K > 256 && K <= 259)), "exl3_shard_cols: shape");
    AMP_REQUIRE(nranges >= 1 && nranges <= SHARD_MAX_RANGES, "exl3_shard_cols: 1..16 ranges");
    AMP_REQUIRE(((uintptr_t) trellis & 15) == 0 && ((uintptr_t) out_trellis & 15) == 0 && ((uintptr_t) svh & 15) == 0 &&
                ((uintptr_t) out_svh & 15) == 0, "exl3_shard_cols: misaligned pointer");
    ShardCols P = {};
    int total = 0;
    for (int i = 0; i < nranges; ++i)
    {
        const int a = ranges[2 * i], len = ranges[2 * i + 1];
        AMP_REQUIRE(a >= 0 && len > 0 && a % 128 == 0 && len % 128 == 0 && (long) a + len <= n,
                    "exl3_shard_cols: range [%d, %d] not 128-aligned/in bounds", a, len);
        P.start[i] = a; P.length[i] = len; P.out_start[i] = total;
        total += len;
    }
    P.trellis = (const unsigned char*) trellis; P.out = (unsigned char*) out_trellis;
    P.svh = (const unsigned char*) svh; P.out_svh = (unsigned char*) out_svh;
    P.tile_bytes = K > 256 ? 16 * (2 * (K - 256) + 1) : 32 * K;        // half-integer rates: 4 * (2 KA + 1) words per tile
    P.nranges = nranges; P.tile_rows = k / 16;
    P.tile_row_bytes_in = (long) (n / 16) * P.tile_bytes; P.tile_row_bytes_out = (long) (total / 16) * P.tile_bytes;
    const int bx = P.tile_rows < 2048 ? P.tile_rows : 2048;
    shard_cols_kernel<<<dim3((unsigned) bx, (unsigned) nranges), 256, 0, stream>>>(P);
    return cuda_rc(cudaGetLastError(), "exl3_shard_cols launch");
}

AMP_API int amp_exl3_shard_rows(const void* trellis, const void* suh, void* out_trellis, void* out_suh, int k, int n, int K,
                                int k0, int klen, cudaStream_t stream)
{
    AMP_REQUIRE(trellis && suh && out_trellis && out_suh, "exl3_shard_rows: null pointer");
    AMP_REQUIRE(k > 0 && n > 0 && k % 16 == 0 && n % 16 == 0 && ((K >= 1 && K <= 8) || (K > 256 && K <= 259)), "exl3_shard_rows: shape");
    AMP_REQUIRE(k0 >= 0 && klen > 0 && k0 % 128 == 0 && klen % 128 == 0 && (long) k0 + klen <= k,
                "exl3_shard_rows: range [%d, %d] not 128-aligned/in bounds", k0, klen);
    const size_t row_bytes = (size_t) (n / 16) * (K > 256 ? 16 * (2 * (K - 256) + 1) : 32 * K);
    if (cudaError_t e = cudaMemcpyAsync(out_trellis, (const unsigned char*) trellis + (size_t) (k0 / 16) * row_bytes,
                                        (size_t) (klen / 16) * row_bytes, cudaMemcpyDefault, stream))
        return cuda_rc(e, "exl3_shard_rows trellis copy");
    return cuda_rc(cudaMemcpyAsync(out_suh, (const unsigned char*) suh + (size_t) k0 * 2, (size_t) klen * 2, cudaMemcpyDefault, stream),
                   "exl3_shard_rows suh copy");
}
