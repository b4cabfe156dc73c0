// Word bindings: op.* and io.* native words that pop their operands from the script stack and
// call the tensor-operator interface.  Stack signatures are the reference's
// (blackriver/nn.cpp:8-371); the leftmost operand is pushed first.
#pragma once

#include "dag.hpp"

namespace br {
void load_nn_words(Enviroment& env);
// value returned by the most recent op.loss_backward word
float last_loss();
}
