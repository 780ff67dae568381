// Lowering of op::Kernel to line-numbered SSA: the restatement of
// ug-core/src/lower_op.rs (index formulas, layout-op folding, reduce lowering,
// Kernel::optimize / lower) plus the compilation-cache key of cache.rs.
#pragma once
#include "ug_core.hpp"

namespace ug {

// lower_op.rs:6-44
struct ThreadBlock { size_t dim = 0, block_dim = 1; };
struct Opts {
  bool has_thread_block = false, has_block_axis = false;
  ThreadBlock thread_block;
  size_t block_axis = 0;
  // Lowering of this backend (not in the reference): reductions over the thread dim are evaluated once,
  // before the loop over that dim, each thread folding its strided share and a ReduceLocal finishing
  // the row.  Needs thread_block.dim == the last dim of the store.
  bool hoist_row_reduces = false;
  Opts with_global_axis(size_t axis, size_t block_dim) const {
    Opts o = *this; o.has_block_axis = true; o.block_axis = axis; o.has_thread_block = true;
    o.thread_block = {axis, block_dim}; return o;
  }
  Opts with_block_axis(size_t axis) const { Opts o = *this; o.has_block_axis = true; o.block_axis = axis; return o; }
  Opts with_thread_block(size_t dim, size_t block_dim) const {
    Opts o = *this; o.has_thread_block = true; o.thread_block = {dim, block_dim}; return o;
  }
};

op::Kernel optimize(op::Kernel k);                      // lower_op.rs:493-535
ssa::Kernel lower(const op::Kernel &k, const Opts &o);  // lower_op.rs:537-557

// cache.rs:8-71: the kernel with its argument ids renumbered 0..n-1, compared structurally.
struct NormalizedKernel {
  std::vector<Arg> args;
  std::vector<op::Store> ops;
  explicit NormalizedKernel(const op::Kernel &k);
  bool operator<(const NormalizedKernel &o) const;
};

}  // namespace ug
