// Packed 4-bit GEMV for large weights: a persistent kernel that keeps the weight stream in flight.
//
// One CTA per SM stays resident. The activation row is staged once per CTA (RMS norm folded
// in). Every warp owns whole 16-row tiles of W and walks them in pieces of up to four 128-column
// blocks; a piece travels global -> shared memory with cp.async (16 bytes per lane and
// instruction for the codes, 4 bytes for the scale pairs) into one of the warp's two ring
// slots, so one piece is always in flight while the other is multiplied. There is no CTA-wide
// synchronisation after the staging: a warp accumulates its tile in registers over all pieces
// and stores its 16 results itself. Tiles are dealt to the warps of the whole grid in a fixed
// order, so the result does not depend on timing.
//
// The multiply is the one of the short-CTA kernel (mma.sync m16n8k16 on exact 136+code
// values, B-column parity separating the two groups of a block, scales applied per group sum).
#include "qgemv_core.cuh"

namespace aoto {

constexpr int STREAM_PIECE_BLOCKS = 4;                          // 128-column blocks per piece
constexpr int STREAM_ROW_PITCH = STREAM_PIECE_BLOCKS * 64 + 64;  // bytes; the pad keeps 128-bit reads conflict-free
constexpr int STREAM_SCALE_OFFSET = 16 * STREAM_ROW_PITCH;       // scale pairs follow the 16 rows
constexpr int STREAM_SLOT_BYTES = STREAM_SCALE_OFFSET + 16 * STREAM_PIECE_BLOCKS * 4;
constexpr int STREAM_MAX_K = 16384;

__device__ __forceinline__ void stream_cp16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void stream_cp4(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1)
qgemv_stream_kernel(const GemvParams p) {
  extern __shared__ uint4 smem[];
  const int K = p.K, N = p.N;
  const int nblocks = K >> 7, groups = K >> 6, chunks = K >> 3;
  uint4* xs = smem;
  uint4* zero16 = xs + chunks;
  float* xsum = reinterpret_cast<float*>(zero16 + 1);
  float* csum = xsum + groups;
  float* red = csum + chunks;
  unsigned char* ring = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(red + 64) + 127) & ~(uintptr_t)127);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tiles = (N + 15) >> 4;
  const int pieces_per_tile = (nblocks + STREAM_PIECE_BLOCKS - 1) / STREAM_PIECE_BLOCKS;
  const int row_bytes = K >> 1;     // packed bytes of a weight row
  const int scale_row = K >> 5;     // bytes of a row of scales
  // tiles are dealt round-robin to the warps of the grid: warp w of CTA c is global warp c + w * grid
  const int global_warp = blockIdx.x + warp * gridDim.x;
  const int global_warps = gridDim.x * WARPS;
  const int my_tiles = tiles > global_warp ? (tiles - global_warp + global_warps - 1) / global_warps : 0;
  const int my_pieces = my_tiles * pieces_per_tile;
  unsigned char* my_ring = ring + (size_t)warp * 2 * STREAM_SLOT_BYTES;
  const unsigned char* wbytes = reinterpret_cast<const unsigned char*>(p.w0);
  const unsigned char* sbytes = reinterpret_cast<const unsigned char*>(p.s0);

  // Request the next piece of this warp (pieces are requested in the order they are consumed:
  // tile after tile, k blocks ascending). Lane pair r copies row r of the tile.
  int req_index = 0, req_tile = 0, req_piece = 0;
  auto request = [&]() {
    if (req_index < my_pieces) {
      const int tile = global_warp + req_tile * global_warps;
      const int kb0 = req_piece * STREAM_PIECE_BLOCKS;
      const int nkb = min(STREAM_PIECE_BLOCKS, nblocks - kb0);
      unsigned char* slot = my_ring + (size_t)(req_index & 1) * STREAM_SLOT_BYTES;
      const int r = lane >> 1;
      const int n = min(tile * 16 + r, N - 1);
      const unsigned char* wsrc = wbytes + (size_t)n * row_bytes + (size_t)kb0 * 64;
      const unsigned char* ssrc = sbytes + (size_t)n * scale_row + (size_t)kb0 * 4;
      for (int j = lane & 1; j < nkb * 4; j += 2) stream_cp16(slot + r * STREAM_ROW_PITCH + j * 16, wsrc + j * 16);
      for (int j = lane & 1; j < nkb; j += 2)
        stream_cp4(slot + STREAM_SCALE_OFFSET + (r * STREAM_PIECE_BLOCKS + j) * 4, ssrc + j * 4);
      ++req_index;
      if (++req_piece == pieces_per_tile) { req_piece = 0; ++req_tile; }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // an empty group keeps the count uniform
  };

  // weights do not depend on the producer of x: start streaming before waiting for it
  request();
  request();
  pdl_wait_for_producers();
  pdl_release_dependents();

  if (tid == 0) *zero16 = make_uint4(0u, 0u, 0u, 0u);
  stage_activation<true>(p, p.x, xs, csum, red);
  for (int gidx = tid; gidx < groups; gidx += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) s += csum[gidx * 8 + c];
    xsum[gidx] = 136.f * s;
  }
  __syncthreads();

  const BSource bs = b_source(xs, zero16, lane);
  float acc_lo = 0.f, acc_hi = 0.f;
  int local_tile = 0, piece = 0;
  for (int index = 0; index < my_pieces; ++index) {
    const int kb0 = piece * STREAM_PIECE_BLOCKS;
    const int nkb = min(STREAM_PIECE_BLOCKS, nblocks - kb0);
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // everything but the newest group has landed
    __syncwarp();
    const unsigned char* slot = my_ring + (size_t)(index & 1) * STREAM_SLOT_BYTES;
#pragma unroll
    for (int j = 0; j < STREAM_PIECE_BLOCKS; ++j) {
      if (j < nkb) {
        WeightItem it;
        it.lo = *reinterpret_cast<const uint4*>(slot + g * STREAM_ROW_PITCH + j * 64 + t * 16);
        it.hi = *reinterpret_cast<const uint4*>(slot + (g + 8) * STREAM_ROW_PITCH + j * 64 + t * 16);
        it.slo = *reinterpret_cast<const uint32_t*>(slot + STREAM_SCALE_OFFSET + (g * STREAM_PIECE_BLOCKS + j) * 4);
        it.shi = *reinterpret_cast<const uint32_t*>(slot + STREAM_SCALE_OFFSET + ((g + 8) * STREAM_PIECE_BLOCKS + j) * 4);
        float lo, hi;
        mma_block(it, bs, kb0 + j, xsum, lo, hi);
        acc_lo += lo;
        acc_hi += hi;
      }
    }
    __syncwarp();        // every lane has read the slot
    request();           // refill it
    if (++piece == pieces_per_tile) {
      piece = 0;
      const int tile = global_warp + local_tile * global_warps;
      if (t == 0) {
        const int n_lo = tile * 16 + g, n_hi = n_lo + 8;
        if (n_lo < N) p.out[n_lo] = __float2bfloat16_rn(finish_output(p, 0, n_lo, acc_lo, 0.f));
        if (n_hi < N) p.out[n_hi] = __float2bfloat16_rn(finish_output(p, 0, n_hi, acc_hi, 0.f));
      }
      acc_lo = acc_hi = 0.f;
      ++local_tile;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

static size_t stream_smem_bytes(int K, int warps) {
  const size_t fixed = (size_t)(K >> 3) * 16 + 16 + (size_t)(K >> 6) * 4 + (size_t)(K >> 3) * 4 + 64 * 4 + 128;
  return fixed + (size_t)warps * 2 * STREAM_SLOT_BYTES;
}

// Only for weights with very many rows (vocabulary-sized): a warp owns whole tiles, so there must
// be a few tiles for every warp of the grid (148 SMs x 16 warps); matrices with fewer rows keep
// the short-CTA kernel, which splits K over the warps of a CTA instead.
bool qgemv_stream_applies(const aoto_qmatmul_args& a) {
  return a.M == 1 && a.group_size == 64 && (a.K % 128) == 0 && a.K <= STREAM_MAX_K &&
         a.epilogue != AOTO_EPILOGUE_SILU_MUL_PAIRED && a.N >= 65536 &&
         (reinterpret_cast<uintptr_t>(a.packed) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.scales) & 3) == 0;
}

int qgemv_stream_launch(const aoto_qmatmul_args& a, cudaStream_t stream) {
  constexpr int WARPS = 16;
  GemvParams p;
  p.x = (const bf16*)a.x;
  p.w0 = (const uint32_t*)a.packed; p.s0 = (const bf16*)a.scales;
  p.w1 = nullptr; p.s1 = nullptr;
  p.addend = (const bf16*)a.addend; p.gate = (const bf16*)a.gate; p.norm_w = (const bf16*)a.norm_weight;
  p.out = (bf16*)a.out;
  p.N = a.N; p.K = a.K; p.group = a.group_size;
  p.addend_kind = a.addend_kind; p.epilogue = a.epilogue;
  p.alpha = a.alpha; p.beta = a.beta; p.eps = a.rms_norm_eps;
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
    (void)cudaGetLastError();
    return AOTO_ERR_LAUNCH;
  }
  static PerDeviceOnce raised;
  if (raise_dynamic_smem(qgemv_stream_kernel<WARPS>, stream_smem_bytes(STREAM_MAX_K, WARPS), raised) != AOTO_OK)
    return AOTO_ERR_LAUNCH;
  const int tiles = (a.N + 15) / 16;
  const int ctas = min(sms, (tiles + WARPS - 1) / WARPS);
  return launch_kernel(qgemv_stream_kernel<WARPS>, dim3(ctas), dim3(WARPS * 32), stream_smem_bytes(a.K, WARPS), stream,
                       (a.flags & AOTO_FLAG_PDL) != 0, p);
}

}  // namespace aoto
