// Stand-in for the reference's `habitat.habitat_cuda` pybind11 module -- TEST
// INFRASTRUCTURE ONLY.  It registers the reference's own bindings
// (cpp/src/frontend/model_bindings.cpp:16-83, compiled from the reference tree)
// and adds the one thing they lack: a way to construct a KernelInstance from
// Python (in the reference, instances only come out of CUPTI profiling,
// cpp/src/habitat_cuda.cpp:15-24).  Used to generate golden fixtures from the
// reference's Python wave-scaling code.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <string>
#include <utility>
#include <vector>

#include "cuda/kernel.h"
#include "frontend/model_bindings.h"

namespace py = pybind11;

PYBIND11_MODULE(habitat_cuda, m) {
  habitat::frontend::bindModels(m);
  m.def("make_kernel",
        [](std::string name, int32_t num_blocks, int32_t block_size, int32_t dynamic_smem,
           int32_t static_smem, int regs, uint64_t run_time_ns,
           std::vector<std::pair<std::string, double>> metrics) {
          habitat::cuda::KernelInstance k(
              habitat::cuda::KernelMetadata(std::move(name), num_blocks, block_size,
                                            dynamic_smem, static_smem,
                                            static_cast<uint16_t>(regs)),
              run_time_ns);
          for (auto& mv : metrics) k.addMetric(mv.first, mv.second);
          return k;
        },
        py::arg("name"), py::arg("num_blocks"), py::arg("block_size"),
        py::arg("dynamic_smem"), py::arg("static_smem"), py::arg("regs"),
        py::arg("run_time_ns"), py::arg("metrics") = std::vector<std::pair<std::string, double>>());
}
