// compile_op: plan an arbitrary N-d redistribution once, execute it many times.
//
// Every rank describes the boxes (offset, shape in global coordinates) it holds as inputs and wants as
// outputs. The planner intersects every output box of this rank with the input boxes of all ranks and
// emits copy pieces; each output element is written exactly once (inputs may overlap — replicated data —
// the first source in preference order wins) and an uncovered element is an error. Pieces are 2-D
// (rows x row_bytes with a source and a destination pitch) so strided intersections such as
// row-sharded -> column-sharded are first-class; the reference's planner computes such pieces too
// (core/processgroup.cc:2848-2984) but its executor only runs byte-contiguous ones
// (core/cputhread.cc:5682-5683).
//
// Execution: on CPU tensors the host engine registers the inputs, announces them and pulls every piece
// with one-sided reads (reference: WorkCustom, core/cputhread.cc:5582-5888). On CUDA tensors the plan is
// lowered to ONE gather/scatter kernel over peer memory (kernels/collectives.cu).
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "host_group.h"

namespace moodist {

struct BoxSpec {
  int rank = 0;
  std::vector<int64_t> offset;
  std::vector<int64_t> shape;
  int64_t numel() const {
    int64_t n = 1;
    for (int64_t s : shape) n *= s;
    return n;
  }
};

struct CopyPiece {
  int src_rank = 0;
  int src_input = 0;    // index among src_rank's inputs
  int dst_output = 0;   // index among this rank's outputs
  uint64_t rows = 1;
  uint64_t row_bytes = 0;
  uint64_t src_offset = 0;  // bytes from the start of the source input tensor
  uint64_t src_pitch = 0;
  uint64_t dst_offset = 0;  // bytes from the start of the destination output tensor
  uint64_t dst_pitch = 0;
};

struct RedistributionPlan {
  int rank = 0, world = 0;
  size_t elem_size = 0;
  std::vector<int64_t> shape;
  std::vector<std::vector<BoxSpec>> inputs;   // [rank] -> that rank's input boxes, in the order given
  std::vector<std::vector<BoxSpec>> outputs;  // [rank]
  std::vector<CopyPiece> pieces;              // what THIS rank copies into its outputs
  std::vector<std::vector<int>> readers;      // [input index of this rank] -> ranks that read it
  std::vector<int> sources;                   // ranks this rank reads from (excluding itself)
  // staging layout for the device path: byte offset of input i of rank r inside r's staging half
  std::vector<std::vector<uint64_t>> stage_offset;
  std::vector<uint64_t> stage_bytes;          // per rank, total staged bytes
};

// Throws moodist::Error on malformed boxes or when an output element has no source.
RedistributionPlan plan_redistribution(const std::vector<int64_t>& shape, size_t elem_size,
                                       const std::vector<BoxSpec>& all_inputs, const std::vector<BoxSpec>& all_outputs,
                                       int rank, int world);

// Host execution of a plan over the engine. One executor per compiled op.
class HostRedistribution {
 public:
  static std::unique_ptr<HostRedistribution> create(HostGroup& group, std::shared_ptr<RedistributionPlan> plan,
                                                    uint32_t op_id);
  virtual ~HostRedistribution() = default;
  // Blocking. inputs[i] / outputs[j]: base pointers of this rank's tensors in plan order.
  virtual void run(const std::vector<const void*>& inputs, const std::vector<void*>& outputs) = 0;
};

}  // namespace moodist
