// Host-side token packing as far as the fused norm kernel needs it: row order, modality tags, and the
// row -> adaLN table index of one denoising step.
//
// Definitions followed (the reference pins them in tests/test_packing.cpp:187-228,416-760 and implements them in
// src/dit/packing.cpp:213-248,407-523; the types are include/slopfab/dit/packing.h:22-73,116-176):
//   * rows are packed [text | condition video | condition audio | audio | video];
//   * index lists: text = the text rows, audio = the audio block, video = every condition row followed by the
//     target video rows; tags: text 1, the audio list 2, the video list 0 (video wins where lists would overlap);
//   * two-timestep step: every row carries the video timestep except the audio list past its conditioning prefix
//     (num_condition_audio entries when the layout says the count is explicit, else num_condition_video), which
//     carries the audio timestep;
//   * four-timestep step (reference-conditioned requests): on top of that the first num_condition_video entries of
//     the video list carry the conditioning-video timestep and the first num_condition_audio entries of the audio
//     list the conditioning-audio timestep;
//   * `unique` is the ascending set of the timesteps that occur (torch.unique semantics: which timestep is index 0
//     flips when two schedules cross), `indices[r]` a row's position in it, adaln[r] = indices[r] * 3 + max(tag[r], 0)
//     -- the clamp keeps padding rows (tag -1) inside the modulation table.
// One routine serves both steps: it materialises the per-row timestep and ranks it against the sorted set.
#include "../../include/sfq.h"

#include <algorithm>
#include <vector>

namespace {

struct Extents {
  int text, cond_video, cond_audio, audio_rows, video_rows;
  bool explicit_audio;
  int condition_start() const { return text; }
  int audio_start() const { return text + cond_video + cond_audio; }
  int video_start() const { return audio_start() + audio_rows; }
  int total() const { return video_start() + video_rows; }
};

bool read_layout(const sfq_sequence_layout* l, Extents& e) {
  if (l == nullptr) return false;
  e = {l->num_text, l->num_condition_video, l->num_condition_audio, l->num_audio_rows, l->num_video_rows,
       l->condition_audio_is_explicit != 0};
  if (e.text < 0 || e.cond_video < 0 || e.cond_audio < 0 || e.audio_rows < 0 || e.video_rows < 0) return false;
  const long long total = (long long)e.text + e.cond_video + e.cond_audio + e.audio_rows + e.video_rows;
  return total <= 0x7FFFFFFF;
}

// Position of row r in the video list (conditions first, then targets), or -1.
int video_list_position(const Extents& e, int r) {
  if (r >= e.condition_start() && r < e.audio_start()) return r - e.condition_start();
  if (r >= e.video_start() && r < e.total()) return (e.audio_start() - e.condition_start()) + (r - e.video_start());
  return -1;
}

void default_tags(const Extents& e, std::vector<int32_t>& tags) {
  tags.assign(size_t(e.total()), 1);
  for (int r = e.audio_start(); r < e.video_start(); ++r) tags[size_t(r)] = 2;
  for (int r = e.condition_start(); r < e.audio_start(); ++r) tags[size_t(r)] = 0;
  for (int r = e.video_start(); r < e.total(); ++r) tags[size_t(r)] = 0;
}

// Ranks every row's timestep in the ascending set of the values that occur and writes the outputs.
int rank_rows(const std::vector<float>& row_t, const int32_t* tags, int32_t* h_indices, int32_t* h_adaln, float* h_unique,
              int unique_capacity, int* h_num_unique) {
  std::vector<float> uniq(row_t);
  std::sort(uniq.begin(), uniq.end());
  uniq.erase(std::unique(uniq.begin(), uniq.end()), uniq.end());
  for (size_t r = 0; r < row_t.size(); ++r) {
    const int32_t idx = int32_t(std::lower_bound(uniq.begin(), uniq.end(), row_t[r]) - uniq.begin());
    if (h_indices) h_indices[r] = idx;
    h_adaln[r] = idx * 3 + std::max(tags[r], int32_t(0));
  }
  if (h_num_unique) *h_num_unique = int(uniq.size());
  if (h_unique)
    for (size_t i = 0; i < uniq.size() && int(i) < unique_capacity; ++i) h_unique[i] = uniq[i];
  return SFQ_OK;
}

}  // namespace

extern "C" {

int sfq_build_indices(const sfq_sequence_layout* layout, int32_t* h_text, int32_t* h_audio, int32_t* h_video, int32_t* h_tags) {
  Extents e;
  if (!read_layout(layout, e)) return SFQ_ERR_INVALID_ARGUMENT;
  if (h_text)
    for (int i = 0; i < e.text; ++i) h_text[i] = i;
  if (h_audio)
    for (int i = 0; i < e.audio_rows; ++i) h_audio[i] = e.audio_start() + i;
  if (h_video) {
    int n = 0;
    for (int r = e.condition_start(); r < e.audio_start(); ++r) h_video[n++] = r;
    for (int r = e.video_start(); r < e.total(); ++r) h_video[n++] = r;
  }
  if (h_tags) {
    std::vector<int32_t> tags;
    default_tags(e, tags);
    std::copy(tags.begin(), tags.end(), h_tags);
  }
  return SFQ_OK;
}

int sfq_build_row_timesteps(const sfq_sequence_layout* layout, const int32_t* h_tags, float video_t, float audio_t,
                            int32_t* h_indices, int32_t* h_adaln, float* h_unique, int unique_capacity, int* h_num_unique) {
  Extents e;
  if (!read_layout(layout, e) || h_adaln == nullptr) return SFQ_ERR_INVALID_ARGUMENT;
  std::vector<int32_t> own;
  if (h_tags == nullptr) {
    default_tags(e, own);
    h_tags = own.data();
  }
  std::vector<float> row_t(size_t(e.total()), video_t);
  const int prefix = std::min(e.explicit_audio ? e.cond_audio : e.cond_video, e.audio_rows);
  for (int r = e.audio_start() + prefix; r < e.video_start(); ++r) row_t[size_t(r)] = audio_t;
  return rank_rows(row_t, h_tags, h_indices, h_adaln, h_unique, unique_capacity, h_num_unique);
}

int sfq_build_row_timesteps4(const sfq_sequence_layout* layout, const int32_t* h_tags, float video_t, float audio_t,
                             float condition_video_t, float condition_audio_t, int32_t* h_indices, int32_t* h_adaln,
                             float* h_unique, int unique_capacity, int* h_num_unique) {
  Extents e;
  if (!read_layout(layout, e) || h_adaln == nullptr) return SFQ_ERR_INVALID_ARGUMENT;
  std::vector<int32_t> own;
  if (h_tags == nullptr) {
    default_tags(e, own);
    h_tags = own.data();
  }
  std::vector<float> row_t(size_t(e.total()), video_t);
  const int video_list = (e.audio_start() - e.condition_start()) + e.video_rows;
  const int cv = std::min(e.cond_video, video_list), ca = std::min(e.cond_audio, e.audio_rows);
  for (int r = 0; r < e.total(); ++r) {
    const int pos = video_list_position(e, r);
    if (pos >= 0 && pos < cv) row_t[size_t(r)] = condition_video_t;
  }
  for (int i = 0; i < e.audio_rows; ++i) row_t[size_t(e.audio_start() + i)] = i < ca ? condition_audio_t : audio_t;
  return rank_rows(row_t, h_tags, h_indices, h_adaln, h_unique, unique_capacity, h_num_unique);
}

int sfq_build_adaln_index(int num_text, int num_condition_video, int num_condition_audio, int condition_audio_is_explicit,
                          int num_audio_rows, int num_video_rows, float video_t, float audio_t, int32_t* h_tags,
                          int32_t* h_indices, int32_t* h_adaln, float* h_unique2, int* h_num_unique) {
  const sfq_sequence_layout l = {num_text, num_condition_video, num_condition_audio, condition_audio_is_explicit,
                                 num_audio_rows, num_video_rows};
  int rc = SFQ_OK;
  if (h_tags != nullptr) rc = sfq_build_indices(&l, nullptr, nullptr, nullptr, h_tags);
  if (rc != SFQ_OK) return rc;
  return sfq_build_row_timesteps(&l, nullptr, video_t, audio_t, h_indices, h_adaln, h_unique2, 2, h_num_unique);
}

}  // extern "C"
