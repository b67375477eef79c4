#include "pyjson.h"
namespace ff { void bind_lowering(py::module &m) {} }
