"""Backend selection and logging: the three environment variables, ``set_backend`` with its
fall-back, and the logger's level / file options (``src/distdl/config.py:8-76`` and
``src/distdl/logger.py`` in the reference)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(code, **env):
    full = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT)
    for k in ("DISTDL_BACKEND_COMM", "DISTDL_BACKEND_ARRAY", "DISTDL_CHECK_INPUT_CHANGED", "DISTDL_LOGLEVEL",
              "DISTDL_LOGFILE"):
        full.pop(k, None)
    full.update(env)
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=180, cwd=ROOT, env=full)
    assert res.returncode == 0, res.stderr[-1500:]
    return res.stdout


REPORT = ("import json, distdl_b200 as d; c = d.config; "
          "print(json.dumps([c.backend_comm, c.backend_array, c.check_input_changed, d.backends.backend.__name__]))")


def test_defaults_without_a_gpu_are_the_cpu_backend():
    comm, array, check, mod = json.loads(_run(REPORT).splitlines()[-1])
    assert (comm, array, check) == ("mpi", "numpy", True) and mod.endswith("cpu_p2p")


def test_environment_variables_select_backend_and_input_check():
    out = _run(REPORT, DISTDL_BACKEND_COMM="nccl", DISTDL_BACKEND_ARRAY="cupy", DISTDL_CHECK_INPUT_CHANGED="0")
    comm, array, check, mod = json.loads(out.splitlines()[-1])
    assert (comm, array, check) == ("nccl", "cupy", False) and mod.endswith("nccl_group")
    # an unknown value falls back to the CPU backend with a warning
    out = _run(REPORT, DISTDL_BACKEND_COMM="smoke-signals", DISTDL_LOGLEVEL="WARNING")
    assert json.loads(out.splitlines()[-1])[0] == "mpi" and "Unknown DISTDL_BACKEND_COMM" in out


def test_set_backend_switches_and_falls_back():
    import distdl_b200 as d
    before = (d.config.backend_comm, d.config.backend_array, d.config.check_input_changed)
    try:
        mod = d.config.set_backend("nccl", "cupy", check_input_changed=False)
        assert d.backends.backend is mod and d.config.backend_comm == "nccl" and not d.config.check_input_changed
        assert d.config.array_is_device()
        mod = d.config.set_backend("native", "torch")                # "torch" is an alias of the device arrays
        assert d.config.backend_array == "cupy" and mod.__name__.endswith("native_b200")
        mod = d.config.set_backend("mpi", "cupy")                    # CUDA-aware MPI has no counterpart: same module
        assert mod.__name__.endswith("cpu_p2p")
        saved = d.backends.supported_backends["nccl_cupy"]
        d.backends.supported_backends["nccl_cupy"] = None            # as after a failed import
        try:
            mod = d.config.set_backend("nccl", "cupy")
            assert (d.config.backend_comm, d.config.backend_array) == ("mpi", "numpy")
        finally:
            d.backends.supported_backends["nccl_cupy"] = saved
        for name in ("Partition", "CartesianPartition", "BufferManager", "ExpandableBuffer", "functional",
                     "get_device", "set_device", "assemble_global_tensor_structure", "broadcast_tensor_structure",
                     "buffer_allocator", "tensor_comm", "tensor_decomposition"):
            assert hasattr(mod, name), name
    finally:
        d.config.set_backend(before[0], before[1], check_input_changed=before[2])


def test_logger_level_and_optional_file(tmp_path):
    code = ("from distdl_b200.logger import logger\n"
            "logger.debug('dbg-line'); logger.warning('warn-line'); logger.error('err-line')\n")
    out = _run(code)                                                   # default level: ERROR on stdout, no file
    assert "err-line" in out and "warn-line" not in out
    assert not os.path.exists(os.path.join(ROOT, "distdl.log"))
    log = tmp_path / "run.log"
    out = _run(code, DISTDL_LOGLEVEL="WARNING", DISTDL_LOGFILE=str(log))
    assert "warn-line" in out and "dbg-line" not in out
    text = log.read_text()
    assert "dbg-line" in text and "err-line" in text and "pid" in text
