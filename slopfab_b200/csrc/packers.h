// Host weight packers (packers.cpp). They throw std::invalid_argument on a contract violation.
#pragma once
#include <cstdint>

namespace sfq {
void pack_nvfp4(const float* w, int out_features, int in_features, float global_scale, uint8_t* data,
                uint8_t* scale_tiled);
void pack_w4a8(const float* w, int out_features, int in_features, int8_t* packed, uint8_t* group_scale,
               float* channel_scale, float* codebook16);
void pack_w6a8(const float* w, int out_features, int in_features, int group, int8_t* packed, uint8_t* group_scale,
               float* channel_scale);
void pack_int8(const float* w, int out_features, int in_features, int convrot_group, int8_t* codes, float* scale);
}  // namespace sfq
