#include "pyjson.h"
namespace ff { void bind_substitutions(py::module &m) {} }
