// Pieces shared by the bf16 tensor-core attention kernels: mma.sync m16n8k16 fragments, ldmatrix, cp.async, the
// XOR swizzle of a [rows][HD] bf16 tile in shared memory, and the paged gather of key / value rows.
#pragma once
#include "common.cuh"

namespace fzattn {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// D (16x8, f32) += A (16x16, bf16, row) * B (16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// 16 bytes global -> shared; with `valid` false the 16 bytes are zero-filled and nothing is read
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *(const uint32_t*)&h;
}

// Byte offset of the 16-byte chunk `chunk` of row `row` in a [rows][HD] bf16 tile: chunks of a row are permuted by the
// row's low three bits, so that the eight rows one ldmatrix reads fall into different banks.
template <int HD>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return (uint32_t)(row * (HD * 2) + ((chunk ^ (row & 7)) << 4));
}

// Gathers keys [key0, key0 + ROWS) of one kv head, keys and values at once, from the paged pools into two swizzled
// [ROWS][HD] tiles. THREADS / ROWS threads share a row: each looks its page up once and copies its part of the key row
// and of the value row (they sit at the same offset of the two pools). Keys outside [lo, hi], or whose page is missing,
// are zero-filled. `trow` is the request's block table.
template <int HD, int ROWS, int THREADS>
__device__ __forceinline__ void load_kv_tile(uint32_t smem_k, uint32_t smem_v, const __nv_bfloat16* __restrict__ k_pool,
                                             const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ trow,
                                             long long page_stride, long long head_off, int page_size, int key0, int lo,
                                             int hi, int tid) {
  constexpr int TPR = THREADS / ROWS;        // threads per row
  constexpr int CHUNKS = HD / 8;             // 16-byte chunks per row
  constexpr int CPT = CHUNKS / TPR;          // chunks per thread
  static_assert(THREADS % ROWS == 0 && CHUNKS % TPR == 0, "tile shape");
  const int r = tid / TPR, c0 = (tid % TPR) * CPT;
  const int key = key0 + r;
  bool valid = key >= lo && key <= hi;
  long long off = 0;
  if (valid) {
    const int pi = key / page_size;
    const int page = trow[pi];
    valid = page >= 0;
    off = (long long)page * page_stride + head_off + (long long)(key - pi * page_size) * HD;
  }
  if (!valid) off = 0;
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    const int c = c0 + i;
    cp_async16(smem_k + swz<HD>(r, c), k_pool + off + c * 8, valid);
    cp_async16(smem_v + swz<HD>(r, c), v_pool + off + c * 8, valid);
  }
}

}  // namespace fzattn
