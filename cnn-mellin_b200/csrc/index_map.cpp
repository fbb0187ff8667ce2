#include "index_map.h"

#include <algorithm>
#include <numeric>
#include <stdexcept>
#include <tuple>

namespace mellin {

bool IndexMapKey::operator<(const IndexMapKey &o) const {
  return std::make_tuple(static_cast<int>(rel), static_cast<int>(sort), nf, ng, nh, s, d, p, u) <
         std::make_tuple(static_cast<int>(o.rel), static_cast<int>(o.sort), o.nf, o.ng, o.nh, o.s, o.d,
                         o.p, o.u);
}

std::vector<Triple> enumerate_triples(Relation rel, int64_t nf, int64_t ng, int64_t nh, int64_t s,
                                      int64_t d, int64_t p, int64_t u) {
  if (p < 0) throw std::invalid_argument("Mellin padding p must be >= 0");
  if (nf < 0 || ng < 0 || nh < 0) throw std::invalid_argument("negative extent");
  if (nf > kIndexMask || ng > kIndexMask || nh > kIndexMask)
    throw std::invalid_argument("Mellin-axis extent does not fit the index tables");
  const int64_t P = p + 1;
  std::vector<Triple> out;
  for (int64_t h = 0; h < nh; ++h) {
    const int64_t t = h + s;
    for (int64_t f = 0; f < nf; ++f) {
      const int64_t k = f + d;
      int64_t num, den;
      if (rel == Relation::Corr) {
        num = t * k;
        den = P;
      } else {
        num = P * t;
        den = k;
      }
      if (den == 0 || num % den != 0) continue;
      const int64_t g = num / den - u;
      if (g < 0 || g >= ng) continue;
      out.push_back(Triple{static_cast<int32_t>(h), static_cast<int32_t>(f), static_cast<int32_t>(g)});
    }
  }
  return out;
}

IndexMap build_index_map(const IndexMapKey &key) {
  std::vector<Triple> triples =
      enumerate_triples(key.rel, key.nf, key.ng, key.nh, key.s, key.d, key.p, key.u);
  IndexMap m;
  m.triples = static_cast<int64_t>(triples.size());
  const int64_t rows = key.sort == SortBy::H ? key.nh : key.sort == SortBy::G ? key.ng : key.nf;
  m.rows = static_cast<int32_t>(rows);
  m.row_ptr.assign(rows + 1, 0);

  auto row_of = [&](const Triple &t) { return key.sort == SortBy::H ? t.h : key.sort == SortBy::G ? t.g : t.f; };

  // For the by-fx order the bias gradient rides along: each hx row of the
  // output gradient must be summed exactly once, so the entry with the
  // smallest fx listing a row "owns" it, and rows no tap reaches are
  // appended to fx = 0 as bias-only entries.
  std::vector<char> owned;
  std::vector<int32_t> orphans;
  if (key.sort == SortBy::F) {
    owned.assign(key.nh, 0);
    for (const Triple &t : triples) owned[t.h] = 1;
    if (key.nf > 0)
      for (int64_t h = 0; h < key.nh; ++h)
        if (!owned[h]) orphans.push_back(static_cast<int32_t>(h));
    std::fill(owned.begin(), owned.end(), 0);
  }

  for (const Triple &t : triples) ++m.row_ptr[row_of(t) + 1];
  if (!orphans.empty()) m.row_ptr[1] += static_cast<int32_t>(orphans.size());
  for (int64_t r = 0; r < rows; ++r) m.row_ptr[r + 1] += m.row_ptr[r];
  m.entries.resize(m.row_ptr[rows]);
  std::vector<int32_t> cursor(m.row_ptr.begin(), m.row_ptr.end() - 1);

  // triples arrive in (h, f) order, so rows come out sorted by h (orders G, F)
  // or by f (order H); for order F the first time a row h is seen is at its
  // smallest f only if we walk by f first -- do that explicitly.
  if (key.sort == SortBy::F || key.sort == SortBy::G) {
    // order G: within a gx row the taps then come in increasing fx, which the
    // tensor-core kernel relies on (weight chunks at increasing addresses)
    std::stable_sort(triples.begin(), triples.end(),
                     [](const Triple &a, const Triple &b) { return a.f < b.f; });
  }
  for (const Triple &t : triples) {
    Entry e;
    switch (key.sort) {
      case SortBy::H: e = Entry{t.f, t.g}; break;
      case SortBy::G: e = Entry{t.f, t.h}; break;
      default:
        e = Entry{t.h, t.g};
        if (!owned[t.h]) {
          owned[t.h] = 1;
          e.a |= kFlagBiasOwner;
        }
        break;
    }
    m.entries[cursor[row_of(t)]++] = e;
  }
  for (int32_t h : orphans) m.entries[cursor[0]++] = Entry{h | kFlagBiasOwner | kFlagBiasOnly, 0};

  m.order.resize(rows);
  std::iota(m.order.begin(), m.order.end(), 0);
  std::stable_sort(m.order.begin(), m.order.end(), [&](int32_t a, int32_t b) {
    return (m.row_ptr[a + 1] - m.row_ptr[a]) > (m.row_ptr[b + 1] - m.row_ptr[b]);
  });
  for (int64_t r = 0; r < rows; ++r) m.max_row = std::max(m.max_row, m.row_ptr[r + 1] - m.row_ptr[r]);
  return m;
}

}  // namespace mellin
