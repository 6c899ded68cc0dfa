// Byte trie over a vocabulary, built on the host and exported as the flat arrays the walk kernel (trie.cu) reads.
//
// Nodes are numbered in creation order (root = 0, then the first token's bytes, ...), exactly as a token-by-token
// insertion into a dictionary trie numbers them, so both builders give identical arrays. Each node keeps its edges
// sorted by byte; a duplicate byte string keeps the lowest id. A 128k-token vocabulary (~0.5 M nodes) builds in tens of
// milliseconds, against seconds for the dictionary version.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <utility>
#include <vector>

namespace {
struct Trie {
  std::vector<std::vector<std::pair<uint8_t, int32_t>>> children;
  std::vector<int32_t> value;
  long long n_edges = 0;
};
}  // namespace

extern "C" {

// blob: the byte strings one behind the other; off[i] .. off[i+1]: string i; ids[i]: its id (strings of length 0 are
// skipped). Returns an opaque handle (null on bad arguments); sizes through n_nodes / n_edges.
void* b200_trie_build(const uint8_t* blob, const long long* off, const int32_t* ids, int n, int* n_nodes,
                      long long* n_edges) {
  if (!off || !ids || n < 0 || !n_nodes || !n_edges || (n > 0 && !blob && off[n] > 0)) return nullptr;
  Trie* t = new Trie();
  t->children.emplace_back();
  t->value.push_back(-1);
  for (int i = 0; i < n; ++i) {
    if (off[i + 1] <= off[i]) continue;
    int32_t node = 0;
    for (long long k = off[i]; k < off[i + 1]; ++k) {
      const uint8_t b = blob[k];
      auto& ch = t->children[node];
      auto it = std::lower_bound(ch.begin(), ch.end(), b,
                                 [](const std::pair<uint8_t, int32_t>& e, uint8_t x) { return e.first < x; });
      if (it != ch.end() && it->first == b) {
        node = it->second;
      } else {
        const int32_t fresh = (int32_t)t->children.size();
        ch.insert(it, std::make_pair(b, fresh));      // `ch` may dangle after the emplace_back below: not used again
        t->children.emplace_back();
        t->value.push_back(-1);
        t->n_edges++;
        node = fresh;
      }
    }
    if (t->value[node] < 0 || ids[i] < t->value[node]) t->value[node] = ids[i];
  }
  *n_nodes = (int)t->children.size();
  *n_edges = t->n_edges;
  return t;
}

// edge_start [n_nodes + 1], edge_byte / edge_child [max(n_edges, 1)], node_value [n_nodes]: caller-allocated.
int b200_trie_export(const void* handle, int32_t* edge_start, uint8_t* edge_byte, int32_t* edge_child,
                     int32_t* node_value) {
  const Trie* t = static_cast<const Trie*>(handle);
  if (!t || !edge_start || !edge_byte || !edge_child || !node_value) return 1;
  long long e = 0;
  for (size_t nidx = 0; nidx < t->children.size(); ++nidx) {
    edge_start[nidx] = (int32_t)e;
    for (const auto& c : t->children[nidx]) {
      edge_byte[e] = c.first;
      edge_child[e] = c.second;
      ++e;
    }
  }
  edge_start[t->children.size()] = (int32_t)e;
  std::memcpy(node_value, t->value.data(), t->value.size() * sizeof(int32_t));
  return 0;
}

void b200_trie_free(void* handle) { delete static_cast<Trie*>(handle); }

}  // extern "C"
