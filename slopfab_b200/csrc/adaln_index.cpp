// Host-side row -> adaLN table index, the integer input of the fused norm kernel.
//
// Follows the definition the reference pins in tests/test_packing.cpp:416-760 and implements in
// src/dit/packing.cpp:213-248,407-489: rows are packed [text | condition video | condition audio | audio |
// video]; every row carries the video timestep except the audio rows past the conditioning prefix, which carry
// the audio timestep; `unique` is the ascending set of the timesteps that occur (torch.unique semantics, so
// which timestep is index 0 flips when the two schedules cross); adaln[r] = index[r] * 3 + max(tag[r], 0)
// with tags video 0, text 1, audio 2.
#include "../../include/sfq.h"

#include <algorithm>
#include <vector>

extern "C" int sfq_build_adaln_index(int num_text, int num_condition_video, int num_condition_audio,
                                     int condition_audio_is_explicit, int num_audio_rows, int num_video_rows,
                                     float video_t, float audio_t, int32_t* h_tags, int32_t* h_indices,
                                     int32_t* h_adaln, float* h_unique2, int* h_num_unique) {
  if (num_text < 0 || num_condition_video < 0 || num_condition_audio < 0 || num_audio_rows < 0 || num_video_rows < 0 ||
      h_adaln == nullptr)
    return SFQ_ERR_INVALID_ARGUMENT;
  const int audio_start = num_text + num_condition_video + num_condition_audio;
  const int video_start = audio_start + num_audio_rows;
  const int total = video_start + num_video_rows;
  // per-row timestep and tag, then the sorted unique set and each row's position in it
  std::vector<float> row_t(size_t(total), video_t);
  std::vector<int32_t> tag(size_t(total), 1);
  for (int r = audio_start; r < video_start; ++r) tag[size_t(r)] = 2;
  for (int r = num_text; r < audio_start; ++r) tag[size_t(r)] = 0;
  for (int r = video_start; r < total; ++r) tag[size_t(r)] = 0;
  const int prefix = std::min(condition_audio_is_explicit ? num_condition_audio : num_condition_video, num_audio_rows);
  for (int r = audio_start + std::max(prefix, 0); r < video_start; ++r) row_t[size_t(r)] = audio_t;
  std::vector<float> uniq(row_t);
  std::sort(uniq.begin(), uniq.end());
  uniq.erase(std::unique(uniq.begin(), uniq.end()), uniq.end());
  for (int r = 0; r < total; ++r) {
    const int32_t idx = int32_t(std::lower_bound(uniq.begin(), uniq.end(), row_t[size_t(r)]) - uniq.begin());
    if (h_indices) h_indices[r] = idx;
    if (h_tags) h_tags[r] = tag[size_t(r)];
    h_adaln[r] = idx * 3 + std::max(tag[size_t(r)], 0);
  }
  if (h_num_unique) *h_num_unique = int(uniq.size());
  if (h_unique2)
    for (size_t i = 0; i < uniq.size() && i < 2; ++i) h_unique2[i] = uniq[i];
  return SFQ_OK;
}
