// Tensor-map construction for the GEMM kernels, with a small cache: the operand tiles
// (bytes, 128-byte swizzle), C / D as 32-bit words, packed fp4 expanded to the padded
// shared-memory form, and the re-laid-out scale atoms.  Included by api.cu only.
#pragma once

#include "host_runtime.h"

namespace {

// ---- tensor maps --------------------------------------------------------------

// The cache consulted below belongs to the device whose lock the calling thread holds;
// the entry points point this at it (DeviceState::tm_cache) before building maps.
thread_local TensorMapSlot* t_tm_cache = nullptr;

TensorMapSlot& tensor_map_slot(const TensorMapKey& k) {
  uint64_t h = k.base * 0x9E3779B97F4A7C15ull;
  h ^= (k.d0 + 0x632BE59BD9B4E019ull) * 0xC2B2AE3D27D4EB4Full;
  h ^= (k.d1 * 31 + k.pitch * 17 + k.box1 * 7 + k.words) * 0x165667B19E3779F9ull;
  return t_tm_cache[(h >> 32) % kTensorMapSlots];
}

// 2-D byte tensor: `inner` contiguous bytes per row, `outer` rows `pitch` bytes
// apart; 128-byte swizzled boxes of box_outer rows; out-of-range reads are zero.
int make_tensor_map(CUtensorMap* tm, const void* base, uint64_t inner, uint64_t outer,
                    uint64_t pitch, uint32_t box_outer) {
  const cuuint64_t dims[2] = {inner, outer};
  if (outer <= 1) pitch = (inner + 15) / 16 * 16;  // a single row: the pitch is never used
  const TensorMapKey key{reinterpret_cast<uint64_t>(base), inner, outer, pitch, box_outer, 0u};
  TensorMapSlot& slot = tensor_map_slot(key);
  if (slot.valid && slot.key == key) {
    *tm = slot.map;
    return 0;
  }
  const cuuint64_t strides[1] = {pitch};
  const cuuint32_t box[2] = {128, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r =
      g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with %d (base %p inner %llu outer %llu pitch %llu box %u)",
              static_cast<int>(r), base, (unsigned long long)inner, (unsigned long long)outer,
              (unsigned long long)pitch, box_outer);
    return CPUOPS_B200_STATUS_CUDA_ERROR;
  }
  slot.valid = true;
  slot.key = key;
  slot.map = *tm;
  return 0;
}

// 2-D tensor of 32-bit words (C): 32 x 32 boxes, 128-byte swizzled rows.
int make_tensor_map_words(CUtensorMap* tm, const void* base, uint64_t cols, uint64_t rows,
                          uint64_t pitch_bytes) {
  const cuuint64_t dims[2] = {cols, rows};
  if (rows <= 1) pitch_bytes = (cols * 4 + 15) / 16 * 16;
  const TensorMapKey key{reinterpret_cast<uint64_t>(base), cols, rows, pitch_bytes, 32u, 1u};
  TensorMapSlot& slot = tensor_map_slot(key);
  if (slot.valid && slot.key == key) {
    *tm = slot.map;
    return 0;
  }
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r =
      g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box,
               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (C) failed with %d", static_cast<int>(r));
    return CPUOPS_B200_STATUS_CUDA_ERROR;
  }
  slot.valid = true;
  slot.key = key;
  slot.map = *tm;
  return 0;
}

// Packed 4-bit rows (k elements, two per byte) read as 128-element boxes that land in
// shared memory in the padded form kind::mxf8f6f4 takes: 16 elements per 16 bytes, so a
// box row is 128 bytes and the 128-byte swizzle applies as for 8-bit operands.  The
// driver requires a 32-byte aligned base and pitch and an inner extent that is a
// multiple of 128 elements: the extent is rounded up, and the caller guarantees that
// the rounded row still lies inside the pitch.
int make_tensor_map_fp4_padded(CUtensorMap* tm, const void* base, uint64_t k_elems, uint64_t outer,
                               uint64_t pitch, uint32_t box_outer) {
  const uint64_t k128 = (k_elems + 127) / 128 * 128;
  if (outer <= 1) pitch = k128 / 2;
  const TensorMapKey key{reinterpret_cast<uint64_t>(base), k128, outer, pitch, box_outer, 3u};
  TensorMapSlot& slot = tensor_map_slot(key);
  if (slot.valid && slot.key == key) {
    *tm = slot.map;
    return 0;
  }
  const cuuint64_t dims[2] = {k128, outer};
  const cuuint64_t strides[1] = {pitch};
  const cuuint32_t box[2] = {128, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r =
      g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), dims, strides,
               box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (padded fp4) failed with %d (base %p k %llu outer %llu pitch %llu)",
              static_cast<int>(r), base, (unsigned long long)k128, (unsigned long long)outer,
              (unsigned long long)pitch);
    return CPUOPS_B200_STATUS_CUDA_ERROR;
  }
  slot.valid = true;
  slot.key = key;
  slot.map = *tm;
  return 0;
}

// The re-laid-out scale array as rows of one 512-byte atom each (128 words, not
// swizzled); a box is the `box_atoms` atoms of one k-block.
int make_tensor_map_atoms(CUtensorMap* tm, const void* base, uint64_t n_atoms, uint32_t box_atoms) {
  const TensorMapKey key{reinterpret_cast<uint64_t>(base), 128, n_atoms, 512, box_atoms, 2u};
  TensorMapSlot& slot = tensor_map_slot(key);
  if (slot.valid && slot.key == key) {
    *tm = slot.map;
    return 0;
  }
  const cuuint64_t dims[2] = {128, n_atoms};
  const cuuint64_t strides[1] = {512};
  const cuuint32_t box[2] = {128, box_atoms};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r =
      g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box,
               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (scale atoms) failed with %d", static_cast<int>(r));
    return CPUOPS_B200_STATUS_CUDA_ERROR;
  }
  slot.valid = true;
  slot.key = key;
  slot.map = *tm;
  return 0;
}

bool tma_addressable(const void* base, int64_t pitch_bytes, int64_t outer) {
  if (reinterpret_cast<uintptr_t>(base) & 15u) return false;
  if (outer > 1 && (pitch_bytes & 15)) return false;
  return true;
}

}  // namespace
