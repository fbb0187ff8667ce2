// Host-side builder of the Mellin index maps.
//
// The Mellin axis couples three indices -- output position hx, kernel tap fx
// and input position gx -- through an exact-divisibility relation (with
// P = p + 1):
//     correlation:  (hx + s)(fx + d) = P (gx + u)      reference: mconv.h:62-66
//     convolution:  P (hx + s)       = (fx + d)(gx + u)  reference: mconv.h:21-26
// Only a sparse, irregular set of (hx, fx, gx) triples satisfies it.  Instead
// of testing divisibility per thread per tap at run time (what the reference
// kernels do, mconv_cuda.cuh:517-554), the triples are enumerated once per
// (relation, extents, s, d, p, u) on the host and stored as a compact CSR
// table in whichever order the consuming kernel walks them:
//     by hx -> forward / operator-level kernels (rows list (fx, gx))
//     by gx -> grad-input kernel                 (rows list (fx, hx))
//     by fx -> grad-weight kernel                (rows list (hx, gx))
// Every index that reaches a kernel has therefore been range-checked here.
#pragma once
#include <cstdint>
#include <vector>

namespace mellin {

enum class Relation : int { Corr = 0, Conv = 1 };
enum class SortBy : int { H = 0, G = 1, F = 2 };

struct Triple {
  int32_t h, f, g;
};

struct IndexMapKey {
  Relation rel;
  SortBy sort;
  int64_t nf, ng, nh, s, d, p, u;
  bool operator<(const IndexMapKey &o) const;
};

// entry flags of the by-fx table, kept in the top bits of Entry::a
constexpr int32_t kFlagBiasOwner = 1 << 29;  // this entry is the first one listing its hx row
constexpr int32_t kFlagBiasOnly = 1 << 30;   // hx row with no tap at all: listed for the bias sum only
constexpr int32_t kIndexMask = (1 << 29) - 1;

struct Entry {
  int32_t a, b;
};

struct IndexMap {
  // CSR over `rows` rows.  Meaning of (a, b) per sort order:
  //   SortBy::H : row = hx, a = fx, b = gx
  //   SortBy::G : row = gx, a = fx, b = hx   (entries of a row in increasing fx)
  //   SortBy::F : row = fx, a = hx | flags, b = gx
  std::vector<int32_t> row_ptr;  // rows + 1
  std::vector<Entry> entries;
  std::vector<int32_t> order;  // rows sorted by decreasing entry count (heaviest first)
  int32_t rows = 0;
  int32_t max_row = 0;  // longest row
  int64_t triples = 0;  // number of (hx, fx, gx) solutions (without bias-only entries)
};

// All solutions with 0 <= h < nh, 0 <= f < nf, 0 <= g < ng, in (h, f) order.
std::vector<Triple> enumerate_triples(Relation rel, int64_t nf, int64_t ng, int64_t nh,
                                      int64_t s, int64_t d, int64_t p, int64_t u);

// Throws std::invalid_argument on extents that do not fit the 29-bit index
// fields or on p < 0.
IndexMap build_index_map(const IndexMapKey &key);

}  // namespace mellin
