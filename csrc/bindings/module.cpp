// Root of the native Python module `kern_b200._native`. Each subsystem registers itself from its
// own translation unit; a subsystem not yet linked into the build is simply absent.
#include <pybind11/pybind11.h>

namespace py = pybind11;

void bind_device(py::module_& m);
#ifdef KERN_WITH_MANIFEST
void bind_manifest(py::module_& m);
#endif
#ifdef KERN_WITH_POOL
void bind_pool(py::module_& m);
#endif
#ifdef KERN_WITH_RUNTIME
void bind_runtime(py::module_& m);
#endif

PYBIND11_MODULE(_native, m) {
  m.doc() = "kern_b200 native core: manifest verifier, pool, device layer, graph executor";
  bind_device(m);
#ifdef KERN_WITH_MANIFEST
  bind_manifest(m);
#endif
#ifdef KERN_WITH_POOL
  bind_pool(m);
#endif
#ifdef KERN_WITH_RUNTIME
  bind_runtime(m);
#endif
}
