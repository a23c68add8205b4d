#include "ndslice/ndslice.h"

#include <algorithm>
#include <cctype>
#include <set>
#include <sstream>

namespace mb {

// -------------------------------------------------------------------------- Slice --
Slice::Slice(size_t offset, std::vector<size_t> sizes, std::vector<size_t> strides)
    : offset_(offset), sizes_(std::move(sizes)), strides_(std::move(strides)) {
  if (sizes_.size() != strides_.size()) throw NdError("sizes and strides differ in length");
  // Reject overlapping layouts: sorted by stride, each stride must clear the span below it.
  std::vector<size_t> order(sizes_.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(),
                   [&](size_t a, size_t b) { return strides_[a] < strides_[b]; });
  size_t span = 0;
  for (size_t i : order) {
    if (sizes_[i] == 0) continue;
    if (sizes_[i] > 1 && strides_[i] <= span && span > 0)
      throw NdError("overlapping slice: stride " + std::to_string(strides_[i]) +
                    " does not clear inner span " + std::to_string(span));
    if (sizes_[i] > 1 && strides_[i] == 0) throw NdError("zero stride on a dimension of size > 1");
    span += (sizes_[i] - 1) * strides_[i];
  }
}

Slice Slice::row_major(const std::vector<size_t>& sizes) {
  std::vector<size_t> strides(sizes.size());
  size_t s = 1;
  for (size_t i = sizes.size(); i-- > 0;) {
    strides[i] = s;
    s *= sizes[i];
  }
  return Slice(0, sizes, strides);
}

size_t Slice::len() const {
  size_t n = 1;
  for (size_t s : sizes_) n *= s;
  return n;
}

bool Slice::is_contiguous() const {
  size_t s = 1;
  for (size_t i = sizes_.size(); i-- > 0;) {
    if (sizes_[i] != 1 && strides_[i] != s) return false;
    s *= sizes_[i];
  }
  return true;
}

size_t Slice::location(const std::vector<size_t>& coords) const {
  if (coords.size() != sizes_.size()) throw NdError("wrong number of coordinates");
  size_t r = offset_;
  for (size_t i = 0; i < coords.size(); ++i) {
    if (coords[i] >= sizes_[i])
      throw NdError("coordinate " + std::to_string(coords[i]) + " out of range for dimension " +
                    std::to_string(i) + " of size " + std::to_string(sizes_[i]));
    r += coords[i] * strides_[i];
  }
  return r;
}

std::vector<size_t> Slice::coordinates(size_t rank) const {
  if (rank < offset_) throw NdError("value " + std::to_string(rank) + " not in slice");
  size_t rem = rank - offset_;
  std::vector<size_t> order(sizes_.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(),
                   [&](size_t a, size_t b) { return strides_[a] > strides_[b]; });
  std::vector<size_t> c(sizes_.size(), 0);
  for (size_t i : order) {
    if (sizes_[i] <= 1 || strides_[i] == 0) continue;
    size_t q = rem / strides_[i];
    if (q >= sizes_[i]) q = sizes_[i] - 1;
    c[i] = q;
    rem -= q * strides_[i];
  }
  if (rem != 0) throw NdError("value " + std::to_string(rank) + " not in slice");
  return c;
}

bool Slice::contains(size_t rank) const {
  try {
    coordinates(rank);
    return true;
  } catch (const NdError&) {
    return false;
  }
}

size_t Slice::get(size_t i) const {
  if (i >= len()) throw NdError("index " + std::to_string(i) + " out of range");
  size_t r = offset_;
  for (size_t d = sizes_.size(); d-- > 0;) {
    r += (i % sizes_[d]) * strides_[d];
    i /= sizes_[d];
  }
  return r;
}

size_t Slice::index(size_t rank) const {
  auto c = coordinates(rank);
  size_t idx = 0;
  for (size_t d = 0; d < sizes_.size(); ++d) idx = idx * sizes_[d] + c[d];
  return idx;
}

std::vector<size_t> Slice::ranks() const {
  std::vector<size_t> out;
  size_t n = len();
  out.reserve(n);
  for (size_t i = 0; i < n; ++i) out.push_back(get(i));
  return out;
}

Slice Slice::at(size_t dim, size_t idx) const {
  if (dim >= sizes_.size()) throw NdError("dimension out of range");
  if (idx >= sizes_[dim]) throw NdError("index out of range");
  auto sz = sizes_, st = strides_;
  size_t off = offset_ + idx * strides_[dim];
  sz.erase(sz.begin() + dim);
  st.erase(st.begin() + dim);
  return Slice(off, sz, st);
}

Slice Slice::select(size_t dim, size_t begin, size_t end, size_t step) const {
  if (dim >= sizes_.size()) throw NdError("dimension out of range");
  if (step == 0) throw NdError("step must be positive");
  end = std::min(end, sizes_[dim]);
  if (begin > end) begin = end;
  auto sz = sizes_, st = strides_;
  sz[dim] = (end - begin + step - 1) / step;
  st[dim] = strides_[dim] * step;
  return Slice(offset_ + begin * strides_[dim], sz, st);
}

Slice Slice::view(const std::vector<size_t>& new_sizes) const {
  size_t n = 1;
  for (size_t s : new_sizes) n *= s;
  if (n != len()) throw NdError("view: element count mismatch");
  if (is_contiguous()) {
    Slice r = row_major(new_sizes);
    return Slice(offset_, r.sizes(), r.strides());
  }
  // General case: greedily map each new dimension onto a run of old dimensions that are
  // mutually contiguous (stride[i] == stride[i+1] * size[i+1]).
  std::vector<size_t> strides(new_sizes.size());
  size_t oi = sizes_.size();
  size_t carry_size = 1, carry_stride = 0;
  for (size_t ni = new_sizes.size(); ni-- > 0;) {
    size_t want = new_sizes[ni];
    if (carry_size == 1) {
      if (oi == 0) {
        if (want != 1) throw NdError("view: incompatible shape");
        strides[ni] = 1;
        continue;
      }
      --oi;
      carry_size = sizes_[oi];
      carry_stride = strides_[oi];
    }
    if (carry_size % want == 0) {
      strides[ni] = carry_stride;
      carry_stride *= want;
      carry_size /= want;
    } else if (want % carry_size == 0) {
      // merge following old dims while contiguous
      size_t have = carry_size;
      size_t base_stride = carry_stride;
      size_t top_stride = carry_stride, top_size = carry_size;
      while (have < want) {
        if (oi == 0) throw NdError("view: incompatible shape");
        --oi;
        if (strides_[oi] != top_stride * top_size) throw NdError("view: not expressible");
        top_stride = strides_[oi];
        top_size = sizes_[oi];
        have *= sizes_[oi];
      }
      if (have != want) throw NdError("view: not expressible");
      strides[ni] = base_stride;
      carry_size = 1;
    } else {
      throw NdError("view: not expressible");
    }
  }
  return Slice(offset_, new_sizes, strides);
}

std::vector<Slice> Slice::from_list(std::vector<size_t> ranks) {
  std::vector<Slice> out;
  if (ranks.empty()) return out;
  std::sort(ranks.begin(), ranks.end());
  ranks.erase(std::unique(ranks.begin(), ranks.end()), ranks.end());
  size_t i = 0;
  while (i < ranks.size()) {
    if (i + 1 == ranks.size()) {
      out.emplace_back(ranks[i], std::vector<size_t>{1}, std::vector<size_t>{1});
      break;
    }
    size_t stride = ranks[i + 1] - ranks[i];
    size_t j = i + 1;
    while (j + 1 < ranks.size() && ranks[j + 1] - ranks[j] == stride) ++j;
    out.emplace_back(ranks[i], std::vector<size_t>{j - i + 1}, std::vector<size_t>{stride});
    i = j + 1;
  }
  return out;
}

std::string Slice::to_string() const {
  std::ostringstream os;
  os << "Slice(offset=" << offset_ << ", sizes=[";
  for (size_t i = 0; i < sizes_.size(); ++i) os << (i ? ", " : "") << sizes_[i];
  os << "], strides=[";
  for (size_t i = 0; i < strides_.size(); ++i) os << (i ? ", " : "") << strides_[i];
  os << "])";
  return os.str();
}

// ------------------------------------------------------------------ Extent / Shape --
size_t Extent::nelements() const {
  size_t n = 1;
  for (size_t s : sizes) n *= s;
  return n;
}
std::string Extent::to_string() const {
  std::ostringstream os;
  os << "{";
  for (size_t i = 0; i < labels.size(); ++i)
    os << (i ? ", " : "") << labels[i] << "=" << sizes[i];
  os << "}";
  return os.str();
}

Shape::Shape(std::vector<std::string> labels, Slice slice)
    : labels_(std::move(labels)), slice_(std::move(slice)) {
  if (labels_.size() != slice_.ndim())
    throw NdError("number of labels (" + std::to_string(labels_.size()) +
                  ") does not match slice dimensions (" + std::to_string(slice_.ndim()) + ")");
  std::set<std::string> seen(labels_.begin(), labels_.end());
  if (seen.size() != labels_.size()) throw NdError("duplicate dimension labels");
}
size_t Shape::dim_of(const std::string& label) const {
  for (size_t i = 0; i < labels_.size(); ++i)
    if (labels_[i] == label) return i;
  throw NdError("invalid label: " + label);
}
Shape Shape::at(const std::string& label, size_t idx) const {
  size_t d = dim_of(label);
  auto l = labels_;
  l.erase(l.begin() + d);
  return Shape(l, slice_.at(d, idx));
}
Shape Shape::select(const std::string& label, size_t begin, size_t end, size_t step) const {
  return Shape(labels_, slice_.select(dim_of(label), begin, end, step));
}
std::map<std::string, size_t> Shape::coordinates(size_t rank) const {
  auto c = slice_.coordinates(rank);
  std::map<std::string, size_t> out;
  for (size_t i = 0; i < c.size(); ++i) out[labels_[i]] = c[i];
  return out;
}
std::string Shape::to_string() const {
  std::ostringstream os;
  os << "{";
  for (size_t i = 0; i < labels_.size(); ++i)
    os << (i ? ", " : "") << labels_[i] << "=" << slice_.sizes()[i];
  os << "}";
  return os.str();
}

// ---------------------------------------------------------------------- Selection --
static Sel mk(Selection::Kind k, Sel a = nullptr, Sel b = nullptr) {
  auto s = std::make_shared<Selection>();
  s->kind = k;
  s->a = std::move(a);
  s->b = std::move(b);
  return s;
}
Sel Selection::f() { static Sel s = mk(False_); return s; }
Sel Selection::t() { static Sel s = mk(True_); return s; }
Sel Selection::all(Sel inner) { return mk(All, std::move(inner)); }
Sel Selection::first(Sel inner) { return mk(First, std::move(inner)); }
Sel Selection::any(Sel inner) { return mk(Any, std::move(inner)); }
Sel Selection::range_of(Range r, Sel inner) {
  auto s = std::make_shared<Selection>();
  s->kind = RangeK;
  s->range = r;
  s->a = std::move(inner);
  return s;
}
Sel Selection::label(std::vector<std::string> l, Sel inner) {
  auto s = std::make_shared<Selection>();
  s->kind = Label;
  s->labels = std::move(l);
  s->a = std::move(inner);
  return s;
}
Sel Selection::intersection(Sel x, Sel y) {
  if (x->kind == False_ || y->kind == False_) return f();
  if (x->kind == True_) return y;
  if (y->kind == True_) return x;
  return mk(Intersection, std::move(x), std::move(y));
}
Sel Selection::union_(Sel x, Sel y) {
  if (x->kind == True_ || y->kind == True_) return t();
  if (x->kind == False_) return y;
  if (y->kind == False_) return x;
  return mk(Union, std::move(x), std::move(y));
}

std::string Selection::to_string() const {
  switch (kind) {
    case False_: return "false";
    case True_: return "true";
    case All: return "all(" + a->to_string() + ")";
    case First: return "first(" + a->to_string() + ")";
    case Any: return "any(" + a->to_string() + ")";
    case Label: return "label(" + a->to_string() + ")";
    case RangeK: {
      std::string r = std::to_string(range.begin) + ":" +
                      (range.end ? std::to_string(*range.end) : "") + ":" +
                      std::to_string(range.step);
      return "range(" + r + ", " + a->to_string() + ")";
    }
    case Intersection: return "intersection(" + a->to_string() + ", " + b->to_string() + ")";
    case Union: return "union(" + a->to_string() + ", " + b->to_string() + ")";
  }
  return "?";
}

// Grammar (lowest to highest precedence):  expr := term ('|' term)* ; term := chain ('&' chain)* ;
// chain := atom (',' chain)? ; atom := '*' | '?' | range | '(' expr ')'.
namespace {
struct Parser {
  const std::string& s;
  size_t i = 0;
  explicit Parser(const std::string& str) : s(str) {}
  void ws() {
    while (i < s.size() && std::isspace((unsigned char)s[i])) ++i;
  }
  bool eat(char c) {
    ws();
    if (i < s.size() && s[i] == c) {
      ++i;
      return true;
    }
    return false;
  }
  [[noreturn]] void fail(const std::string& why) {
    throw NdError("selection parse error at " + std::to_string(i) + " in '" + s + "': " + why);
  }
  std::optional<size_t> number() {
    ws();
    size_t j = i;
    size_t v = 0;
    while (j < s.size() && std::isdigit((unsigned char)s[j])) v = v * 10 + (s[j++] - '0');
    if (j == i) return std::nullopt;
    i = j;
    return v;
  }
  // Replace the terminal `true` leaves of `s` by `cont`.
  static Sel append(const Sel& s, const Sel& cont) {
    switch (s->kind) {
      case Selection::True_: return cont;
      case Selection::False_: return s;
      case Selection::All: return Selection::all(append(s->a, cont));
      case Selection::First: return Selection::first(append(s->a, cont));
      case Selection::Any: return Selection::any(append(s->a, cont));
      case Selection::RangeK: return Selection::range_of(s->range, append(s->a, cont));
      case Selection::Label: return Selection::label(s->labels, append(s->a, cont));
      case Selection::Union: return Selection::union_(append(s->a, cont), append(s->b, cont));
      case Selection::Intersection:
        return Selection::intersection(append(s->a, cont), append(s->b, cont));
    }
    return s;
  }
  // Applies `inner` to a parsed dimension atom.
  using Wrap = std::function<Sel(Sel)>;
  Sel expr() {
    Sel l = term();
    while (eat('|')) l = Selection::union_(l, term());
    return l;
  }
  Sel term() {
    Sel l = chain();
    while (eat('&')) l = Selection::intersection(l, chain());
    return l;
  }
  Sel chain() {
    ws();
    if (eat('(')) {
      Sel e = expr();
      if (!eat(')')) fail("expected ')'");
      // "(a|b),rest": the continuation applies below every branch of the group
      if (eat(',')) return append(e, chain());
      return e;
    }
    Wrap w;
    if (eat('*')) {
      w = [](Sel in) { return Selection::all(in); };
    } else if (eat('?')) {
      w = [](Sel in) { return Selection::any(in); };
    } else {
      Range r;
      auto b = number();
      ws();
      if (i < s.size() && s[i] == ':') {
        ++i;
        r.begin = b.value_or(0);
        r.end = number();
        ws();
        if (i < s.size() && s[i] == ':') {
          ++i;
          auto st = number();
          if (st) {
            if (*st == 0) fail("step must be positive");
            r.step = *st;
          }
        }
      } else {
        if (!b) fail("expected '*', '?', a number, a range or '('");
        r.begin = *b;
        r.end = *b + 1;
      }
      w = [r](Sel in) { return Selection::range_of(r, in); };
    }
    if (eat(',')) return w(chain());
    return w(Selection::t());
  }
};
}  // namespace

Sel Selection::parse(const std::string& text) {
  Parser p(text);
  Sel r = p.expr();
  p.ws();
  if (p.i != text.size()) p.fail("trailing input");
  return r;
}

Sel Selection::of_ranks(const Slice& slice, const std::vector<size_t>& ranks) {
  Sel acc = f();
  for (size_t r : ranks) {
    auto c = slice.coordinates(r);
    Sel s = t();
    for (size_t d = c.size(); d-- > 0;) s = range_of(Range{c[d], c[d] + 1, 1}, s);
    acc = union_(acc, s);
  }
  return acc;
}

bool accepts_leaf(const Sel& sel) {
  switch (sel->kind) {
    case Selection::False_: return false;
    case Selection::True_: return true;
    case Selection::Union: return accepts_leaf(sel->a) || accepts_leaf(sel->b);
    case Selection::Intersection: return accepts_leaf(sel->a) && accepts_leaf(sel->b);
    default: return accepts_leaf(sel->a);
  }
}

static bool maybe_nonempty(const Sel& sel) {
  switch (sel->kind) {
    case Selection::False_: return false;
    case Selection::Union: return maybe_nonempty(sel->a) || maybe_nonempty(sel->b);
    case Selection::Intersection: return maybe_nonempty(sel->a) && maybe_nonempty(sel->b);
    case Selection::True_: return true;
    default: return maybe_nonempty(sel->a);
  }
}

std::vector<std::pair<size_t, Sel>> expand(const Sel& sel, size_t n, std::mt19937_64& rng) {
  std::vector<std::pair<size_t, Sel>> out;
  switch (sel->kind) {
    case Selection::False_: break;
    case Selection::True_:
      for (size_t i = 0; i < n; ++i) out.emplace_back(i, sel);
      break;
    case Selection::All:
      for (size_t i = 0; i < n; ++i) out.emplace_back(i, sel->a);
      break;
    case Selection::RangeK: {
      size_t end = std::min(sel->range.end.value_or(n), n);
      for (size_t i = sel->range.begin; i < end; i += sel->range.step) out.emplace_back(i, sel->a);
      break;
    }
    case Selection::First:
      if (n > 0 && maybe_nonempty(sel->a)) out.emplace_back(0, sel->a);
      break;
    case Selection::Any:
      if (n > 0) out.emplace_back((size_t)(rng() % n), sel->a);
      break;
    case Selection::Label: return expand(sel->a, n, rng);
    case Selection::Union: {
      auto x = expand(sel->a, n, rng), y = expand(sel->b, n, rng);
      std::map<size_t, Sel> m;
      for (auto& [i, s] : x) m[i] = m.count(i) ? Selection::union_(m[i], s) : s;
      for (auto& [i, s] : y) m[i] = m.count(i) ? Selection::union_(m[i], s) : s;
      for (auto& kv : m) out.emplace_back(kv.first, kv.second);
      break;
    }
    case Selection::Intersection: {
      auto x = expand(sel->a, n, rng), y = expand(sel->b, n, rng);
      std::map<size_t, Sel> mx;
      for (auto& [i, s] : x) mx[i] = mx.count(i) ? Selection::union_(mx[i], s) : s;
      std::map<size_t, Sel> m;
      for (auto& [i, s] : y) {
        auto it = mx.find(i);
        if (it == mx.end()) continue;
        Sel z = Selection::intersection(it->second, s);
        if (z->kind == Selection::False_) continue;
        m[i] = m.count(i) ? Selection::union_(m[i], z) : z;
      }
      for (auto& kv : m) out.emplace_back(kv.first, kv.second);
      break;
    }
  }
  return out;
}

static void eval_rec(const Sel& sel, const Slice& slice, size_t dim, size_t base,
                     std::mt19937_64& rng, std::vector<size_t>& out) {
  if (dim == slice.ndim()) {
    if (accepts_leaf(sel)) out.push_back(base);
    return;
  }
  for (auto& [i, rest] : expand(sel, slice.sizes()[dim], rng))
    eval_rec(rest, slice, dim + 1, base + i * slice.strides()[dim], rng, out);
}

std::vector<size_t> eval(const Sel& sel, const Slice& slice, uint64_t seed) {
  std::mt19937_64 rng(seed);
  std::vector<size_t> out;
  eval_rec(sel, slice, 0, slice.offset(), rng, out);
  std::vector<size_t> dedup;
  std::set<size_t> seen;
  for (size_t r : out)
    if (seen.insert(r).second) dedup.push_back(r);
  return dedup;
}

// ------------------------------------------------------------------------ routing --
RoutingFrame RoutingFrame::root(Sel sel, const Slice& slice) {
  RoutingFrame f;
  f.here.assign(slice.ndim(), 0);
  f.sel = std::move(sel);
  f.dim = 0;
  return f;
}

Resolved resolve_routing(size_t rank, const Slice& slice, std::vector<RoutingFrame> frames,
                         uint64_t seed) {
  Resolved out;
  std::mt19937_64 rng(seed ^ (0x9E3779B97F4A7C15ull * (rank + 1)));
  while (!frames.empty()) {
    RoutingFrame f = std::move(frames.back());
    frames.pop_back();
    if (f.dim == slice.ndim()) {
      if (accepts_leaf(f.sel)) out.deliver_here = true;
      continue;
    }
    for (auto& [i, rest] : expand(f.sel, slice.sizes()[f.dim], rng)) {
      RoutingFrame nf;
      nf.here = f.here;
      nf.here[f.dim] = i;
      nf.sel = rest;
      nf.dim = f.dim + 1;
      size_t peer = slice.location(nf.here);
      if (peer == rank)
        frames.push_back(std::move(nf));
      else
        out.next[peer].push_back(std::move(nf));
    }
  }
  return out;
}

Slice reshape_with_limit(const Slice& slice, size_t limit) {
  if (limit < 2) return slice;
  std::vector<size_t> sizes, strides;
  for (size_t d = 0; d < slice.ndim(); ++d) {
    size_t n = slice.sizes()[d], st = slice.strides()[d];
    if (n <= limit) {
      sizes.push_back(n);
      strides.push_back(st);
      continue;
    }
    // Factor n into chunks <= limit, largest usable factor first.
    std::vector<size_t> factors;
    size_t rem = n;
    while (rem > limit) {
      size_t f = 0;
      for (size_t c = limit; c >= 2; --c)
        if (rem % c == 0) {
          f = c;
          break;
        }
      if (f == 0) break;  // prime remainder above the limit: keep as is
      factors.push_back(f);
      rem /= f;
    }
    factors.push_back(rem);
    // row-major over the factors: last factor is innermost
    size_t inner = st;
    std::vector<size_t> fs(factors.size());
    for (size_t i = factors.size(); i-- > 0;) {
      fs[i] = inner;
      inner *= factors[i];
    }
    for (size_t i = 0; i < factors.size(); ++i) {
      sizes.push_back(factors[i]);
      strides.push_back(fs[i]);
    }
  }
  return Slice(slice.offset(), sizes, strides);
}

}  // namespace mb
