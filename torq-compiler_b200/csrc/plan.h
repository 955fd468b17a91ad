// Launch planning: turns the op records of a torq-b200-ops blob into a list of
// ready-to-launch steps, lays the intermediate activations out in one arena by
// liveness, and assembles the image of derived constants (packed weights,
// per-channel epilogue parameters) that is uploaded once per executable - the
// counterpart of the reference loading its code/constant segments once in
// TorqExecutable::initialize (runtime/driver/TorqExecutable.cc:1138-1178).
#pragma once
#include <cuda_runtime.h>

#include <functional>
#include <string>
#include <vector>

#include "../../include/torq_b200_ops.h"

namespace tb200 {

struct ExecContext {
  char* arena;
  char* consts;
  void* const* io;  // inputs then outputs
  cudaStream_t stream;
  int* status;      // device status word (0 = fine)
  char* scratch;    // per-dispatch scratch shared by the ops that need one (split-K partials, ...)
  char* const* peer_scratch;  // tensor parallelism: every rank's scratch area as mapped here, or null
  cudaError_t* launch_error;  // a step whose launcher refuses (not a CUDA launch failure) records why here
};

// Where a tensor lives at dispatch time.
struct Loc {
  enum Kind { ARENA, IO, CONST, NONE } kind = NONE;
  size_t offset = 0;  // byte offset in arena / const image, or io index
  void* resolve(const ExecContext& c) const {
    switch (kind) {
      case ARENA: return c.arena + offset;
      case CONST: return c.consts + offset;
      case IO: return c.io[offset];
      default: return nullptr;
    }
  }
};

struct Step {
  const char* kernel_name = "";
  int launches = 1;
  std::function<void(const ExecContext&)> launch;
};

struct Plan {
  std::vector<Step> steps;        // one per op, in order
  std::vector<uint8_t> const_image;
  size_t arena_bytes = 0;
  size_t state_bytes = 0;         // prefix of the arena holding persistent state, zeroed at create
  size_t launch_count = 0;
  size_t scratch_offset = 0;      // scratch sits behind the activations inside the arena allocation
  size_t scratch_bytes = 0;
  bool zero_scratch = false;      // the scratch must read as zero before the first dispatch
  bool use_graph = true;          // replay the launch list as a CUDA graph
  int tp = 1, rank = 0;           // tensor-parallel group size and this executable's place in it
  std::vector<Loc> tensor_loc;
};

// Returns a tb200_status value; `err` holds the message on failure.
int build_plan(const std::vector<tb200_tensor_t>& tensors, const std::vector<tb200_op_t>& ops,
               const std::vector<uint8_t>& constants, Plan& plan, std::string& err);

}  // namespace tb200
