// Monotonic alignment search: for every sequence, the assignment of frames to tokens that maximises the summed score
// over paths where frame 0 takes token 0, the last frame the last token, and the token index never decreases nor
// skips. One CTA per sequence, threads over the tokens: a frame's row of best totals needs only the previous row, so two
// rows ping-pong in shared memory (global scratch when a row does not fit); per cell one byte records whether the best
// predecessor was the previous token. Thread 0 then walks back from the last frame and writes the 0 / 1 path.
// Ties keep the same token (the host version in audio/vits.py makes the same choice).
//
// Reference counterpart: the alignment step of the speech trainer's VITS mode (src/Idrak.Audio).
#include "common.cuh"

namespace idrak {

constexpr int kAlignThreads = 256;
constexpr int kAlignSmemTokens = 6000;       // two fp32 rows of this many tokens stay under 48 KB
constexpr float kAlignNeg = -1e30f;

// score [B, F, T]; frames, tokens [B]; path [B, F, T] (zeroed by the caller); step [B, F, T] bytes; rows [B, 2, T].
__global__ void __launch_bounds__(kAlignThreads) align_kernel(const float* __restrict__ score,
                                                              const int* __restrict__ frames,
                                                              const int* __restrict__ tokens, float* __restrict__ path,
                                                              unsigned char* __restrict__ step, float* __restrict__ rows,
                                                              int F, int T, int use_smem) {
  extern __shared__ float smem[];
  const int b = blockIdx.x;
  const int Fb = min(frames[b], F), Tb = min(tokens[b], T);
  if (Fb < 1 || Tb < 1 || Fb < Tb) return;
  float* row[2];
  row[0] = use_smem ? smem : rows + size_t(b) * 2 * T;
  row[1] = row[0] + T;
  const float* sc = score + size_t(b) * F * T;
  unsigned char* st = step + size_t(b) * F * T;
  for (int f = 0; f < Fb; ++f) {
    const float* prev = row[(f + 1) & 1];
    float* cur = row[f & 1];
    for (int t = threadIdx.x; t < Tb; t += blockDim.x) {
      float v = kAlignNeg;
      unsigned char moved = 0;
      if (f == 0) {
        if (t == 0) v = sc[0];
      } else if (t <= f) {
        const float stay = prev[t];
        const float diag = t > 0 ? prev[t - 1] : kAlignNeg;
        moved = diag > stay;
        v = fmaxf(sc[size_t(f) * T + t] + fmaxf(stay, diag), kAlignNeg);
      }
      cur[t] = v;
      st[size_t(f) * T + t] = moved;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    float* pb = path + size_t(b) * F * T;
    int idx = Tb - 1;
    for (int f = Fb - 1; f >= 0; --f) {
      pb[size_t(f) * T + idx] = 1.f;
      if (f > 0 && idx > 0 && (idx == f || st[size_t(f) * T + idx])) --idx;
    }
  }
}

}  // namespace idrak

using namespace idrak;

IDRAK_API int idrak_monotonic_align(const float* score, const int* frames, const int* tokens, float* path,
                                    unsigned char* step, float* rows, int B, int F, int T, void* stream_) {
  if (B < 1 || F < 1 || T < 1) return -2;
  const int use_smem = T <= kAlignSmemTokens;
  const size_t smem = use_smem ? size_t(2) * T * sizeof(float) : 0;
  align_kernel<<<B, kAlignThreads, smem, static_cast<cudaStream_t>(stream_)>>>(score, frames, tokens, path, step, rows,
                                                                               F, T, use_smem);
  note_launches(1);
  return int(cudaGetLastError());
}
