// Autograd-graph analysis for the incremental gradient generator.
//
// Parity: python/monarch/gradient/_gradient_generator.cpp (the incremental executor that
// hands gradients out one at a time in backward order) and gradient_generator.py
// (gradient_execution_order).  Here the stock autograd engine runs the backward on its own
// thread and tensor hooks publish each gradient the moment it is final; this extension
// supplies what needs the C++ graph API: the order in which those gradients will become
// available, and the set of graph nodes a gradient depends on (used to size buckets).
#include <torch/extension.h>
#include <torch/csrc/autograd/function.h>
#include <torch/csrc/autograd/functions/accumulate_grad.h>

#include <algorithm>
#include <limits>
#include <queue>
#include <unordered_map>
#include <unordered_set>

using torch::autograd::Edge;
using torch::autograd::Node;

namespace {

Edge gradient_edge(const at::Tensor& t) {
  if (auto fn = t.grad_fn()) return Edge(fn, t.output_nr());
  return Edge(torch::autograd::impl::grad_accumulator(t), 0);
}

struct EdgeKey {
  Node* node;
  uint32_t nr;
  bool operator==(const EdgeKey& o) const { return node == o.node && nr == o.nr; }
};
struct EdgeHash {
  size_t operator()(const EdgeKey& k) const {
    return std::hash<void*>()(k.node) * 31 + k.nr;
  }
};

// Reverse order of each tensor's first use in the backward computation: the engine runs
// nodes by descending sequence number, so a gradient is final once the consumer with the
// smallest sequence number has run.
std::vector<int64_t> execution_order(const std::vector<at::Tensor>& roots,
                                     const std::vector<at::Tensor>& wrt) {
  std::unordered_map<EdgeKey, double, EdgeHash> min_seq;
  std::vector<EdgeKey> keys;
  std::vector<std::shared_ptr<Node>> keep;  // keep accumulators alive while we look
  for (auto& t : wrt) {
    TORCH_CHECK(t.requires_grad(), "gradient_execution_order: tensor does not require grad");
    Edge e = gradient_edge(t);
    keep.push_back(e.function);
    EdgeKey k{e.function.get(), e.input_nr};
    keys.push_back(k);
    min_seq[k] = std::numeric_limits<double>::infinity();
  }
  std::vector<Node*> stack;
  for (auto& r : roots) {
    Edge e = gradient_edge(r);
    keep.push_back(e.function);
    if (e.function) stack.push_back(e.function.get());
  }
  std::unordered_set<Node*> seen;
  while (!stack.empty()) {
    Node* n = stack.back();
    stack.pop_back();
    if (!seen.insert(n).second) continue;
    for (const Edge& e : n->next_edges()) {
      if (!e.function) continue;
      stack.push_back(e.function.get());
      auto it = min_seq.find(EdgeKey{e.function.get(), e.input_nr});
      if (it != min_seq.end())
        it->second = std::min(it->second, (double)n->sequence_nr());
    }
  }
  std::vector<int64_t> order(wrt.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = (int64_t)i;
  std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) {
    return min_seq[keys[a]] > min_seq[keys[b]];
  });
  return order;
}

// Number of autograd nodes reachable from `roots` (graph size; used by tests/diagnostics).
int64_t graph_size(const std::vector<at::Tensor>& roots) {
  std::vector<Node*> stack;
  std::vector<std::shared_ptr<Node>> keep;
  for (auto& r : roots) {
    Edge e = gradient_edge(r);
    keep.push_back(e.function);
    if (e.function) stack.push_back(e.function.get());
  }
  std::unordered_set<Node*> seen;
  while (!stack.empty()) {
    Node* n = stack.back();
    stack.pop_back();
    if (!seen.insert(n).second) continue;
    for (const Edge& e : n->next_edges())
      if (e.function) stack.push_back(e.function.get());
  }
  return (int64_t)seen.size();
}

}  // namespace

PYBIND11_MODULE(_gradgen, m) {
  m.def("execution_order", &execution_order);
  m.def("graph_size", &graph_size);
}
