/*
 * Upstream keeps its enums and structs in include/xnor_nn_types.h and its functions in
 * include/xnor_nn.h. Here both live in xnor_nn.h; this header exists so that code which includes
 * "xnor_nn_types.h" by name keeps compiling.
 */
#ifndef XNOR_NN_TYPES_H
#define XNOR_NN_TYPES_H
#include "xnor_nn.h"
#endif
