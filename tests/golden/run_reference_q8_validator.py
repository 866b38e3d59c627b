"""Runs the reference project's own block-32 validation script, unmodified, against the C checker.

  python tests/golden/run_reference_q8_validator.py /path/to/reference

The reference validates its block-32 (Q8_0) W8A8 kernel with benchmarks/benchmark_q8_block_int8.py:
it loads a shared library with ctypes, calls the raw entry point ``q8_block_int8(x, a, sa, w, sw, y,
m, n, k, stream)`` on three shapes (a zero block and a block scaled by 100 among them), captures the
call in a CUDA graph, replays it on negated inputs and asserts — scales within rtol 1e-6 of
``absmax/127``, every code within 0.50002 of the exact quotient, the output within rtol 0.008 of its
blockwise FP32 formula, and a relative error below 0.015 against the dense product (lines 86-113).
The script holds no vectors: it draws its inputs at run time and needs a GPU.

This runner executes that script's ``main`` as it is, on a machine without a GPU, against
oracle/libci8_oracle.so, whose ``q8_block_int8`` is the host twin of the reference's entry point. Two
stand-ins make that possible and nothing else is touched:
  * the script's ``torch`` name resolves to a thin proxy that builds "cuda" tensors on the CPU and
    offers stand-ins for torch.cuda's stream, event and graph objects; a "graph" records the raw
    library calls made while it is captured and issues them again on replay, with the same baked-in
    pointers, which is what a CUDA graph of this script does;
  * the script's ``ctypes.CDLL`` hands out the real library with the entry point wrapped so that the
    recorder sees the calls.
Every assertion of the reference's script then runs on the checker's outputs. The result (the
script's own JSON records, minus timings) is written to q8_block_validator.json next to this file:
it pins the C checker — and with it the torch checker and the CUDA kernel, which are compared with it
bit for bit elsewhere — to the reference's own acceptance test for this path.
"""
import ctypes
import hashlib
import importlib.util
import json
import sys
import tempfile
import time
import types
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
SCRIPT = Path("benchmarks") / "benchmark_q8_block_int8.py"


class _Recorder:
    """What a capturing graph sees: the library calls issued while it is open."""

    def __init__(self):
        self.capturing = None


class _Graph:
    def __init__(self):
        self.calls = []

    def replay(self):
        for function, arguments in self.calls:
            assert function(*arguments) == 0


class _Capture:
    def __init__(self, recorder, graph):
        self.recorder, self.graph = recorder, graph

    def __enter__(self):
        self.recorder.capturing = self.graph

    def __exit__(self, *exc):
        self.recorder.capturing = None
        return False


class _Event:
    def __init__(self, enable_timing=False):
        self.at = 0.0

    def record(self):
        self.at = time.perf_counter()

    def synchronize(self):
        pass

    def elapsed_time(self, other):
        return (other.at - self.at) * 1e3


class _Entry:
    """The library's entry point; argtypes / restype go to the real function."""

    def __init__(self, function, recorder):
        object.__setattr__(self, "_function", function)
        object.__setattr__(self, "_recorder", recorder)

    def __setattr__(self, name, value):
        setattr(self._function, name, value)

    def __call__(self, *arguments):
        if self._recorder.capturing is not None:
            self._recorder.capturing.calls.append((self._function, arguments))
        return self._function(*arguments)


def _torch_proxy(recorder):
    def on_cpu(factory):
        def build(*args, **kwargs):
            if kwargs.get("device") == "cuda":
                kwargs["device"] = "cpu"
            return factory(*args, **kwargs)
        return build

    cuda = types.SimpleNamespace(
        set_device=lambda index: None,
        current_stream=lambda: types.SimpleNamespace(cuda_stream=0),
        CUDAGraph=_Graph,
        graph=lambda graph: _Capture(recorder, graph),
        Event=_Event,
        get_device_properties=lambda index: "host stand-in (no GPU)",
    )

    class Proxy:
        def __getattr__(self, name):
            return getattr(torch, name)

    proxy = Proxy()
    proxy.cuda = cuda
    for name in ("empty", "zeros", "randn", "randint"):
        setattr(proxy, name, on_cpu(getattr(torch, name)))
    return proxy


def _ctypes_proxy(recorder):
    class Library:
        def __init__(self, path):
            self._library = ctypes.CDLL(path)

        def __getattr__(self, name):
            return _Entry(getattr(self._library, name), recorder)

    class Proxy:
        CDLL = Library

        def __getattr__(self, name):
            return getattr(ctypes, name)

    return Proxy()


def run(reference_root: Path, library: Path) -> dict:
    script = reference_root / SCRIPT
    spec = importlib.util.spec_from_file_location("reference_q8_validator", script)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)          # defines main(); nothing runs yet
    recorder = _Recorder()
    module.torch = _torch_proxy(recorder)
    module.ctypes = _ctypes_proxy(recorder)
    with tempfile.TemporaryDirectory() as scratch:
        output = Path(scratch) / "report.jsonl"
        arguments = types.SimpleNamespace(library=library, entry="q8_block_int8", manifest=None, native_library=None,
                                          compare_b12x=False, output=output, device=0, rows=[128])
        module.main(arguments)               # raises AssertionError if any of the reference's checks fails
        records = [json.loads(line) for line in output.read_text().splitlines()]
    kept = ("m", "n", "k", "relative_l2", "candidate_relative_l2", "entry", "scope", "weight_requantization")
    return dict(
        reference_script=str(SCRIPT),
        reference_script_sha256=hashlib.sha256(script.read_bytes()).hexdigest(),
        library="oracle/libci8_oracle.so (host twin of the reference's q8_block_int8)",
        torch=torch.__version__,
        passed=True,
        shapes=[{key: record[key] for key in kept} for record in records],
    )


def main():
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    import subprocess

    subprocess.run(["make", "-s", "-C", str(ROOT / "oracle")], check=True)
    result = run(Path(sys.argv[1]).resolve(), ROOT / "oracle" / "libci8_oracle.so")
    (HERE / "q8_block_validator.json").write_text(json.dumps(result, indent=1) + "\n")
    print(json.dumps(result))


if __name__ == "__main__":
    main()
