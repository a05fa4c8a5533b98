// Helpers shared by the IR passes and the code generators.
#pragma once
#include <vector>

#include "cogito.h"

namespace cgjit {
bool is_elementwise(cg_ir_opcode op);
bool is_binary(cg_ir_opcode op);
bool is_reduction(cg_ir_opcode op);
int tensor_size(const cg_ir_graph* g, int tensor_id);
// tensor id -> indices of the live nodes that read it
std::vector<std::vector<int>> consumers(const cg_ir_graph* g);
bool is_graph_output(const cg_ir_graph* g, int tensor_id);
}  // namespace cgjit
