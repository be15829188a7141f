// Additive Python bindings beside ormi-core's own module (which is built unchanged): the two pointwise functions its
// binding file leaves out although the ops exist (ormi-core/csrc/bindings/bind_pointwise.cpp:16-25 binds add, sub, mul,
// div, sin, cos, neg, exp; core/ops/pointwise/log.h and pow.h are there too), and the backend's own switches, which
// ormi-core has no API for.  Import ormi_backend first: the Node type is registered there.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>

#include "core/node.h"
#include "core/ops/pointwise/log.h"
#include "core/ops/pointwise/pow.h"
#include "b200_backend.h"

namespace py = pybind11;

PYBIND11_MODULE(ormi_backend_extra, m) {
    m.doc() = "log / pow function bindings and B200 backend switches beside ormi_backend";
    m.def("log", &ormi::ops::log);
    m.def("pow", &ormi::ops::pow);
    m.def("set_device", [](int device) { ormi::cuda::set_active_device(device); },
          "device that later CUDA allocations (and the graphs built on them) go to; one process per GPU sets its local rank");
    m.def("active_device", [] { return ormi::cuda::active_device(); });
    m.def("set_option", [](const std::string& key, const std::string& value) {
        if (ormi_b200_set_option(ormi::cuda::b200_context(), key.c_str(), value.c_str()) != 0) throw std::runtime_error(ormi_b200_last_error());
    });
    m.def("counter", [](const std::string& name) {
        int64_t v = 0;
        if (ormi_b200_get_counter(ormi::cuda::b200_context(), name.c_str(), &v) != 0) throw std::runtime_error(ormi_b200_last_error());
        return v;
    });
}
