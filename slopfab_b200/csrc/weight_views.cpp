// Views over a row-fused weight: the k-th of `parts` equal row blocks of a [parts * rows_each, in_features] weight,
// e.g. Wq / Wk / Wv of the canonical contiguous [Wq; Wk; Wv] upload.
//
// Follows build_block of the reference (src/dit/transformer_load.cpp:660-737): every array that is indexed by weight
// row moves with the view -- the packed data, the group / block scales and the per-channel scales -- because
// advancing `data` alone gives finite, well-shaped and wrong results. The offsets are byte offsets only where each
// block is a whole number of the storage units involved:
//   NVFP4   block scales live in 128-row tiles, so rows_each must be a multiple of 128;
//   NF4     a block must be a whole number of absmax blocks and of nested blocks;
//   W4A8 / W6A8  group scales are row-major [N, K / group], channel scales [N]; W6 rows are K * 3 / 4 bytes.
// Pointers may be host or device pointers; nothing is dereferenced.
#include "../../include/sfq.h"

#include <cstddef>
#include <cstdint>

namespace {
const uint8_t* bytes(const void* p) { return static_cast<const uint8_t*>(p); }
}  // namespace

extern "C" int sfq_weight_row_block(const sfq_quant_weight* fused, int parts, int index, sfq_quant_weight* out) {
  if (fused == nullptr || out == nullptr || parts <= 0 || index < 0 || index >= parts || fused->out_features <= 0 ||
      fused->in_features <= 0 || fused->out_features % parts != 0 || fused->data == nullptr)
    return SFQ_ERR_INVALID_ARGUMENT;
  const size_t rows = size_t(fused->out_features) / size_t(parts);
  const size_t k = size_t(fused->in_features);
  const size_t elems = rows * k;  // elements of one block
  sfq_quant_weight v = *fused;
  v.out_features = int32_t(rows);
  const size_t at = size_t(index);
  switch (fused->format) {
    case SFQ_W4A8:
    case SFQ_W6A8: {
      const size_t group = fused->packed_group_size;
      if (group == 0 || k % group != 0 || fused->block_scale == nullptr || fused->weight_scale == nullptr)
        return SFQ_ERR_INVALID_ARGUMENT;
      v.data = bytes(fused->data) + at * (elems * (fused->format == SFQ_W6A8 ? 6 : 4) / 8);
      v.block_scale = fused->block_scale + at * (elems / group);
      v.weight_scale = fused->weight_scale + at * rows;
      break;
    }
    case SFQ_NF4: {
      const size_t block = size_t(fused->nf4_block_size), nested = size_t(fused->nf4_nested_block_size);
      if (block == 0 || nested == 0 || elems % block != 0 || (elems / block) % nested != 0 || elems % 2 != 0 ||
          fused->nf4_absmax == nullptr || fused->nf4_nested_absmax == nullptr)
        return SFQ_ERR_INVALID_ARGUMENT;  // "qkv thirds do not align to NF4 nested blocks"
      v.data = bytes(fused->data) + at * (elems / 2);
      v.nf4_absmax = fused->nf4_absmax + at * (elems / block);
      v.nf4_nested_absmax = fused->nf4_nested_absmax + at * (elems / block / nested);
      break;
    }
    case SFQ_NVFP4: {
      // the scale tile index runs row-major over 128-row tiles: a block that starts mid-tile cannot be addressed
      if (rows % 128 != 0 || k % 16 != 0 || fused->block_scale == nullptr) return SFQ_ERR_INVALID_ARGUMENT;
      v.data = bytes(fused->data) + at * (elems / 2);
      v.block_scale = fused->block_scale + at * (elems / 16);
      break;
    }
    case SFQ_F32:
    case SFQ_F16:
    case SFQ_BF16:
    case SFQ_F8E4M3:
    case SFQ_I8: {
      const size_t width = fused->format == SFQ_F32 ? 4 : (fused->format == SFQ_F16 || fused->format == SFQ_BF16 ? 2 : 1);
      v.data = bytes(fused->data) + at * elems * width;
      if (fused->per_channel_scale && fused->weight_scale != nullptr) v.weight_scale = fused->weight_scale + at * rows;
      break;
    }
    default:
      return SFQ_ERR_INVALID_ARGUMENT;
  }
  if (fused->bias != nullptr) {
    if (fused->bias_format != SFQ_F32 && fused->bias_format != SFQ_BF16) return SFQ_ERR_INVALID_ARGUMENT;
    v.bias = bytes(fused->bias) + at * rows * (fused->bias_format == SFQ_F32 ? 4 : 2);
  }
  *out = v;
  return SFQ_OK;
}
