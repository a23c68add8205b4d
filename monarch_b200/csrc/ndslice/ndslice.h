// N-dimensional strided index sets (Slice), labelled shapes, points, and the selection
// algebra with its text grammar and cast-tree routing.
//
// Parity: ndslice/src/slice.rs (Slice), shape.rs (Shape, select/at), view.rs
// (Extent/Point), selection.rs + selection/parse.rs (Selection, grammar),
// selection/routing.rs (RoutingFrame::next_steps, resolve_routing), reshape.rs
// (reshape_with_limit).
//
// Design: selections are evaluated and routed through one primitive, `expand`, the
// per-dimension derivative of a selection: the list of (index, residual selection)
// pairs it admits in the current dimension.  Evaluation is a DFS over `expand`;
// routing sends each residual to the node that owns that index.  Because both use
// the same primitive, "routing delivers exactly the evaluated set, once" holds by
// construction.
#pragma once
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <optional>
#include <random>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace mb {

struct NdError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class Slice {
 public:
  Slice() : offset_(0) {}
  Slice(size_t offset, std::vector<size_t> sizes, std::vector<size_t> strides);
  static Slice row_major(const std::vector<size_t>& sizes);
  // Decompose an arbitrary rank list into maximal strided slices.
  static std::vector<Slice> from_list(std::vector<size_t> ranks);

  size_t offset() const { return offset_; }
  const std::vector<size_t>& sizes() const { return sizes_; }
  const std::vector<size_t>& strides() const { return strides_; }
  size_t ndim() const { return sizes_.size(); }
  size_t len() const;
  bool is_contiguous() const;

  // coordinates -> flat rank
  size_t location(const std::vector<size_t>& coords) const;
  // flat rank -> coordinates (throws if the rank is not in the slice)
  std::vector<size_t> coordinates(size_t rank) const;
  // i-th element (row-major enumeration) -> flat rank
  size_t get(size_t i) const;
  // flat rank -> position in the row-major enumeration
  size_t index(size_t rank) const;
  bool contains(size_t rank) const;
  std::vector<size_t> ranks() const;

  // Fix dimension `dim` to `idx` (dimension is dropped).
  Slice at(size_t dim, size_t idx) const;
  // Restrict dimension `dim` to [begin, end) with step.
  Slice select(size_t dim, size_t begin, size_t end, size_t step) const;
  // A row-major view of the same elements with new sizes (product must match and the
  // slice must be expressible); throws otherwise.
  Slice view(const std::vector<size_t>& new_sizes) const;

  bool operator==(const Slice& o) const {
    return offset_ == o.offset_ && sizes_ == o.sizes_ && strides_ == o.strides_;
  }
  std::string to_string() const;

 private:
  size_t offset_;
  std::vector<size_t> sizes_, strides_;
};

struct Extent {
  std::vector<std::string> labels;
  std::vector<size_t> sizes;
  size_t nelements() const;
  std::string to_string() const;
  bool operator==(const Extent& o) const { return labels == o.labels && sizes == o.sizes; }
};

class Shape {
 public:
  Shape() = default;
  Shape(std::vector<std::string> labels, Slice slice);
  const std::vector<std::string>& labels() const { return labels_; }
  const Slice& slice() const { return slice_; }
  size_t dim_of(const std::string& label) const;
  Shape at(const std::string& label, size_t idx) const;
  Shape select(const std::string& label, size_t begin, size_t end, size_t step) const;
  std::map<std::string, size_t> coordinates(size_t rank) const;
  Extent extent() const { return Extent{labels_, slice_.sizes()}; }
  std::string to_string() const;
  bool operator==(const Shape& o) const { return labels_ == o.labels_ && slice_ == o.slice_; }

 private:
  std::vector<std::string> labels_;
  Slice slice_;
};

// ---------------------------------------------------------------------- Selection --
struct Selection;
using Sel = std::shared_ptr<const Selection>;

struct Range {
  size_t begin = 0;
  std::optional<size_t> end;
  size_t step = 1;
};

struct Selection {
  enum Kind { False_, True_, All, First, RangeK, Any, Label, Intersection, Union } kind;
  Range range;                       // RangeK
  std::vector<std::string> labels;   // Label
  Sel a, b;                          // inner (a) / operands (a,b)

  static Sel f();
  static Sel t();
  static Sel all(Sel inner);
  static Sel first(Sel inner);
  static Sel any(Sel inner);
  static Sel range_of(Range r, Sel inner);
  static Sel label(std::vector<std::string> l, Sel inner);
  static Sel intersection(Sel x, Sel y);
  static Sel union_(Sel x, Sel y);
  // Text grammar: `*` all, `?` any, `3` index, `1:4`, `0:8:2`, `:`; `,` descends to the
  // next dimension; `|` union; `&` intersection; parentheses.
  static Sel parse(const std::string& text);
  // Selection matching exactly `ranks` of `slice`.
  static Sel of_ranks(const Slice& slice, const std::vector<size_t>& ranks);
  std::string to_string() const;
};

// The (index, residual) pairs `sel` admits in a dimension of size n.  `rng` supplies the
// randomness of `?`; deterministic given the seed.
std::vector<std::pair<size_t, Sel>> expand(const Sel& sel, size_t n, std::mt19937_64& rng);
// Whether `sel` accepts a fully-addressed element (no dimensions left).
bool accepts_leaf(const Sel& sel);
// All flat ranks of `slice` matched by `sel`, in row-major order (deduplicated).
std::vector<size_t> eval(const Sel& sel, const Slice& slice, uint64_t seed = 4);

// ------------------------------------------------------------------------ routing --
// A cast travels down a tree rooted at the slice's first element: the node holding a
// frame at dimension d owns coordinates here[0..d) (later coordinates are 0) and
// forwards, for each admitted index i of dimension d, the residual selection to the node
// at (here[0..d), i, 0, ...).
struct RoutingFrame {
  std::vector<size_t> here;
  Sel sel;
  size_t dim = 0;

  static RoutingFrame root(Sel sel, const Slice& slice);
};

struct Resolved {
  bool deliver_here = false;
  std::map<size_t, std::vector<RoutingFrame>> next;  // peer rank -> frames to forward
};

// Process the frames that arrived at `rank`: expand locally while the next hop is this
// same rank, collect frames for other ranks.
Resolved resolve_routing(size_t rank, const Slice& slice, std::vector<RoutingFrame> frames,
                         uint64_t seed = 4);

// Split dimensions larger than `limit` into factors <= limit (row-major), so that a cast
// tree over the reshaped slice has bounded fan-out.  The element set is unchanged.
Slice reshape_with_limit(const Slice& slice, size_t limit);

}  // namespace mb
