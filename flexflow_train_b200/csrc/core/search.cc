#include "pyjson.h"
namespace ff { void bind_search(py::module &m) {} }
