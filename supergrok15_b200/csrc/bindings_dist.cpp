#include "bindings_decl.h"
namespace sgb { void register_dist(pybind11::module_& m) {} }
