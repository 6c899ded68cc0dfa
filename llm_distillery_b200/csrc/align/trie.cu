// Byte-trie walk for cross-tokenizer alignment.
//
// The student vocabulary is a trie over the byte strings of its tokens, stored flat: node n owns the edges
// edge_start[n] .. edge_start[n+1]-1, sorted by byte; edge e leads to node edge_child[e]; node_value[n] is the student
// token whose byte string ends at n (-1: none). One thread walks one teacher token's bytes from the root and keeps
// the value of the deepest node that is a token: the student token that is the LONGEST prefix of the teacher token,
// i.e. what a greedy longest-match tokenizer would emit first. The result is the teacher-id -> student-id table that
// remap_topk (csrc/loss/topk_logprob.cu) sends every collected row through.
//
// Memory-latency bound: a walk is a chain of dependent lookups (a binary search over at most 256 sorted edges per
// byte), so the kernel relies on many independent walks in flight - one per thread, a whole vocabulary per launch.
#include <cstdint>

#include "../common/host.cuh"

namespace b200 {
namespace align {

__global__ void __launch_bounds__(256) trie_walk_kernel(const int* __restrict__ edge_start,
                                                       const uint8_t* __restrict__ edge_byte,
                                                       const int* __restrict__ edge_child,
                                                       const int* __restrict__ node_value, int n_nodes,
                                                       const uint8_t* __restrict__ tok_bytes,
                                                       const long long* __restrict__ tok_off, int n_tokens,
                                                       int* __restrict__ out, int* __restrict__ out_len) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens) return;
  int node = 0, best = -1, best_len = 0;
  const long long b0 = tok_off[t], b1 = tok_off[t + 1];
  for (long long i = b0; i < b1; ++i) {
    const uint8_t b = tok_bytes[i];
    int lo = edge_start[node];
    const int end = edge_start[node + 1];
    int hi = end;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (edge_byte[mid] < b) lo = mid + 1;
      else hi = mid;
    }
    if (lo >= end || edge_byte[lo] != b) break;
    node = edge_child[lo];
    if (node <= 0 || node >= n_nodes) break;      // malformed table: stop rather than read outside it
    const int v = node_value[node];
    if (v >= 0) {
      best = v;
      best_len = (int)(i - b0) + 1;
    }
  }
  out[t] = best;
  if (out_len) out_len[t] = best_len;
}

}  // namespace align
}  // namespace b200

// out[t] = student token that is the longest byte-prefix of teacher token t (-1: none); out_len[t] (optional) = how
// many bytes of the teacher token that student token covers.
extern "C" int b200_trie_walk(const int* edge_start, const uint8_t* edge_byte, const int* edge_child,
                              const int* node_value, int n_nodes, const uint8_t* tok_bytes, const long long* tok_off,
                              int n_tokens, int* out, int* out_len, cudaStream_t st) {
  using namespace b200;
  if (!edge_start || !edge_byte || !edge_child || !node_value || !tok_bytes || !tok_off || !out || n_nodes <= 0 ||
      n_tokens <= 0)
    return B200_ERR_ARG;
  align::trie_walk_kernel<<<(n_tokens + 255) / 256, 256, 0, st>>>(edge_start, edge_byte, edge_child, node_value, n_nodes,
                                                                  tok_bytes, tok_off, n_tokens, out, out_len);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
