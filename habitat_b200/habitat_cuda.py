"""Host-side mirror of the reference's `habitat.habitat_cuda` pybind11 module.

Same class and property names as cpp/src/frontend/model_bindings.cpp:16-83 of
the reference (DeviceProperties, KernelInstance), so code written against the
reference's bindings keeps working.  Two differences:
  * KernelInstance can be constructed from Python (in the reference, instances
    only come out of CUPTI profiling, cpp/src/habitat_cuda.cpp:15-24);
  * thread_block_occupancy() runs the batched sm_100a kernel on one record; the
    reference runs NVIDIA's occupancy header on the host.
"""
import ctypes

from habitat_b200 import _native


class DeviceProperties:
    """cpp/src/cuda/kernel.h:14-62, bound at cpp/src/frontend/model_bindings.cpp:17-55."""

    def __init__(self, name, compute_major, compute_minor, max_threads_per_block,
                 max_threads_per_multiprocessor, regs_per_block, regs_per_multiprocessor,
                 warp_size, shared_mem_per_block, shared_mem_per_multiprocessor, num_sms,
                 shared_mem_per_block_optin, mem_bandwidth_gb, base_clock_mhz,
                 peak_gflops_per_second, reserved_shared_mem_per_block=None):
        self._name = str(name)
        if reserved_shared_mem_per_block is None:
            # the driver reserves 1 KiB of shared memory per block from cc 8.0 on
            reserved_shared_mem_per_block = 1024 if int(compute_major) >= 8 else 0
        values = dict(
            compute_major=compute_major, compute_minor=compute_minor,
            max_threads_per_block=max_threads_per_block,
            max_threads_per_multiprocessor=max_threads_per_multiprocessor,
            regs_per_block=regs_per_block, regs_per_multiprocessor=regs_per_multiprocessor,
            warp_size=warp_size, shared_mem_per_block=shared_mem_per_block,
            shared_mem_per_multiprocessor=shared_mem_per_multiprocessor, num_sms=num_sms,
            shared_mem_per_block_optin=shared_mem_per_block_optin,
            reserved_shared_mem_per_block=reserved_shared_mem_per_block,
            mem_bandwidth_gb=mem_bandwidth_gb, base_clock_mhz=base_clock_mhz,
            peak_gflops_per_second=peak_gflops_per_second)
        for key, value in values.items():
            if int(value) != value:
                raise TypeError("%s must be an integer, got %r" % (key, value))
        self._fields = {k: int(v) for k, v in values.items()}

    def __repr__(self):
        return "DeviceProperties(name=" + self._name + ")"

    @property
    def name(self):
        return self._name

    @property
    def num_sms(self):
        return self._fields["num_sms"]

    @property
    def mem_bandwidth_gb(self):
        return self._fields["mem_bandwidth_gb"]

    @property
    def compute_capability(self):
        return (self._fields["compute_major"], self._fields["compute_minor"])

    @property
    def base_clock_mhz(self):
        return self._fields["base_clock_mhz"]

    @property
    def peak_gflops_per_second(self):
        return self._fields["peak_gflops_per_second"]

    def spec_tuple(self):
        """The fifteen integers of an hb_device_spec, in declaration order."""
        return tuple(self._fields[f] for f in _native.DEVICE_SPEC_FIELDS)


class KernelInstance:
    """cpp/src/cuda/kernel.h:64-151, bound at cpp/src/frontend/model_bindings.cpp:57-82."""

    def __init__(self, name, num_blocks, block_size, dynamic_shared_memory=0,
                 static_shared_memory=0, registers_per_thread=0, run_time_ns=0, metrics=()):
        self._name = str(name)
        self._num_blocks = int(num_blocks)
        self._block_size = int(block_size)
        self._dynamic_shared_memory = int(dynamic_shared_memory)
        self._static_shared_memory = int(static_shared_memory)
        self._registers_per_thread = int(registers_per_thread) & 0xFFFF  # uint16_t in the reference
        self._run_time_ns = int(run_time_ns)
        self._metrics = [(str(n), float(v)) for n, v in metrics]

    @property
    def name(self):
        return self._name

    @property
    def run_time_ns(self):
        return self._run_time_ns

    @property
    def num_blocks(self):
        return self._num_blocks

    @property
    def metrics(self):
        return self._metrics

    @property
    def metadata(self):
        return dict(
            name=self._name, num_blocks=self._num_blocks, block_size=self._block_size,
            static_shared_memory=self._static_shared_memory,
            dynamic_shared_memory=self._dynamic_shared_memory,
            registers_per_thread=self._registers_per_thread)

    def launch_record(self):
        """(name, num_blocks, block_size, registers_per_thread, static + dynamic shared memory,
        run_time_ns): the fields wave scaling reads, without building the metadata dict."""
        return (self._name, self._num_blocks, self._block_size, self._registers_per_thread,
                self._static_shared_memory + self._dynamic_shared_memory, self._run_time_ns)

    def add_metric(self, name, value):
        self._metrics.append((str(name), float(value)))

    def thread_block_occupancy(self, device, registers_per_thread=-1):
        """Active thread blocks per SM on `device`; 0 if the launch cannot run there."""
        from habitat_b200 import device_table
        regs = self._registers_per_thread if registers_per_thread < 0 else int(registers_per_thread) & 0xFFFF
        row = device_table.row_of(device)
        occ = ctypes.c_int32(0)
        limits = (ctypes.c_int32 * 4)()
        smem = self._dynamic_shared_memory + self._static_shared_memory
        if smem < 0 or self._block_size < 0 or self._block_size > 0xFFFF:
            return 0
        lib = _native.load()
        _native.check(lib.hb_thread_block_occupancy(
            row, self._block_size, smem, regs, ctypes.byref(occ), limits))
        return int(occ.value)
