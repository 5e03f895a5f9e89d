// TEST INFRASTRUCTURE.  Stand-in for the reference's include/common/common.h when its host MLP
// (test/mlp.h) is compiled on its own: that header only needs the Activation enum (same
// enumerator order as include/common/common.h:28-38) and a few standard headers it forgets.
#pragma once
#include <algorithm>
#include <iomanip>
#include <stdexcept>
enum class Activation { ReLU, LeakyReLU, Exponential, Sine, Sigmoid, Squareplus, Softplus, Tanh, None };
