// Internal interface of the sampling tail (sampler.cu) for the decoder.
#pragma once

#include "../../include/b200step.h"
#include "common.cuh"

namespace b200 {

constexpr int SAMPLE_TOPK_ROUNDS_MAX = 64;   // up to this K the K largest are picked by K passes; above, by a full sort

// Device bytes sample_rows needs for `rows` rows of V logits under cfg (0 for greedy).
size_t sample_workspace_bytes(const b200_sampling& cfg, int V, int rows);
// True when cfg never reaches a random draw (Sampler::sample's first branch).
bool sampling_is_greedy(const b200_sampling& cfg);

// One Sampler::sample per row, enqueued on the current stream.  The token history of row r is
// the ring hist[r * cap .. + cap): totals[r] tokens were pushed in all, token number j (from 0)
// sits at j % cap, the newest min(totals[r], cap) are available.  ws: device scratch of
// sample_workspace_bytes.  logits are modified in place (penalties, bans) like the reference's.
int sample_rows(float* logits, int V, int rows, const int32_t* hist, int cap, const int32_t* totals,
                const b200_sampling& cfg, uint64_t* rng, int32_t* next, void* ws);

// hist[r] <- tokens[r] appended (ring), totals[r] += 1, for every row.
int history_push(int32_t* hist, int cap, int32_t* totals, const int32_t* tokens, int rows);
// The prompt: tokens [rows, T] appended row by row; with seq_off (device, [rows + 1]) row r's
// tokens are tokens[seq_off[r] .. seq_off[r + 1]) and T is ignored.
int history_push_prompt(int32_t* hist, int cap, int32_t* totals, const int32_t* tokens, int rows, int T,
                        const int32_t* seq_off = nullptr);

// Sum over rows with a target in [0, V) of logZ - logit[target] (+ z * logZ^2), added to
// acc[0] (double) and the number of such rows to acc[1] (as a double-sized int64); losses:
// device scratch of n doubles.  A target >= V sets acc[2] (int64) non-zero.
int cross_entropy_accumulate(const float* logits, const int32_t* targets, int64_t n, int V, float z_scale, double* losses,
                             double* acc);

}  // namespace b200
