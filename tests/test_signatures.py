"""The argument types that the Python side declares for the library's entry points must be
the ones in the CUDA sources: a pointer passed as an int would be cut to 32 bits."""
import re
from pathlib import Path

import nimbus_infer_rs_b200.csrc as csrc_pkg
from nimbus_infer_rs_b200.csrc.signatures import SIGNATURES

OTHER = {"nb_last_error", "nb_attention_decode_static_capacity"}   # declared by hand (results)


def _letters(arg: str) -> str:
    arg = arg.strip()
    if "*" in arg or "cudaStream_t" in arg:
        return "p"
    for prefix, letter in (("float", "f"), ("double", "d"), ("long long", "l"), ("int", "i"),
                           ("const int", "i")):
        if arg.startswith(prefix + " "):
            return letter
    raise AssertionError(f"argument type not understood: {arg!r}")


def test_declared_signatures_match_the_sources():
    found = {}
    for path in sorted(Path(csrc_pkg.__file__).parent.glob("*.cu")):
        text = path.read_text()
        for m in re.finditer(r"NB_EXPORT\s+[\w\s\*]+?\s+(\w+)\s*\(([^)]*)\)", text):
            args = [a for a in " ".join(m.group(2).split()).split(",") if a.strip()]
            found[m.group(1)] = "".join(_letters(a) for a in args)
    assert found, "no entry points found"
    for name, letters in found.items():
        if name in OTHER:
            assert letters == ""
            continue
        assert SIGNATURES.get(name) == letters, name
    assert set(SIGNATURES) == set(found) - OTHER


# Kernel parameters that point to constants of the model: the only ones that may be
# `__restrict__` in a kernel that can start before its predecessor has ended.
CONSTANT_PARAMS = {"gamma", "beta", "bias", "W", "wte", "wpe"}


def test_no_restrict_on_step_data_in_kernels_that_start_early():
    """A kernel that calls nb_grid_dependency_wait() may start while the kernel before it still
    runs.  Loads through a `const __restrict__` pointer are invariant to the compiler, which may
    move them in front of that wait, where the predecessor has not written the data yet (it
    happened to the decode attention's query rows).  So in such kernels only pointers to
    constants carry the qualifier."""
    src_dir = Path(csrc_pkg.__file__).parent
    checked = 0
    for path in sorted(list(src_dir.glob("*.cu")) + list(src_dir.glob("*.cuh"))):
        text = path.read_text()
        for m in re.finditer(r"__global__[^;{]*?(\w+)\s*\(([^)]*)\)\s*\{", text, re.S):
            name, params = m.group(1), m.group(2)
            # the kernel's body: up to the next kernel or the end of the file
            nxt = text.find("__global__", m.end())
            body = text[m.end(): nxt if nxt >= 0 else len(text)]
            if "nb_grid_dependency_wait" not in body:
                continue
            checked += 1
            for p in params.split(","):
                if "__restrict__" in p:
                    pname = p.strip().split()[-1]
                    assert pname in CONSTANT_PARAMS, f"{path.name}: {name}({pname}) is __restrict__"
    assert checked >= 15


def test_the_cpu_stand_in_has_the_signatures_of_the_cuda_backend():
    """The host-logic tests run the engine on `tests/cpu_backend.py`; what they prove about the
    engine holds on the GPU only if both backends are called the same way."""
    import inspect

    import cpu_backend
    from nimbus_infer_rs_b200.csrc.ops import CudaBackend

    stand_in = next(c for _, c in inspect.getmembers(cpu_backend, inspect.isclass)
                    if c.__module__ == cpu_backend.__name__ and hasattr(c, "linear"))
    checked = 0
    for name, fn in inspect.getmembers(stand_in, inspect.isfunction):
        if name.startswith("_"):
            continue
        real = getattr(CudaBackend, name, None)
        assert real is not None, f"CudaBackend has no method {name}"
        mine, theirs = inspect.signature(fn), inspect.signature(real)
        assert list(mine.parameters) == list(theirs.parameters), name
        for k, p in mine.parameters.items():
            q = theirs.parameters[k]
            assert (p.default is inspect.Parameter.empty) == (q.default is inspect.Parameter.empty), (name, k)
        checked += 1
    assert checked >= 12


def test_every_call_into_the_library_passes_as_many_arguments_as_declared():
    """ctypes would take a call with an argument too few or too many and the kernel would read
    what lies beside them; count the arguments of every ``_call("nb_...", ...)`` and
    ``lib.nb_...(...)`` in the package against the declared signatures."""
    import ast

    root = Path(csrc_pkg.__file__).parent.parent
    seen = set()
    for path in sorted(root.rglob("*.py")):
        for node in ast.walk(ast.parse(path.read_text())):
            if not isinstance(node, ast.Call) or any(isinstance(a, ast.Starred) for a in node.args):
                continue
            f = node.func
            if isinstance(f, ast.Attribute) and f.attr == "_call" and node.args \
                    and isinstance(node.args[0], ast.Constant):
                name, n = node.args[0].value, len(node.args) - 1
            elif isinstance(f, ast.Attribute) and f.attr.startswith("nb_"):
                name, n = f.attr, len(node.args)
            else:
                continue
            if name in OTHER:
                continue
            assert name in SIGNATURES, f"{path.name}:{node.lineno}: {name} is not declared"
            assert n == len(SIGNATURES[name]), f"{path.name}:{node.lineno}: {name} takes {len(SIGNATURES[name])}"
            # and a pointer stands exactly where a pointer is declared
            for kind, arg in zip(SIGNATURES[name], node.args[len(node.args) - n:]):
                pointer = isinstance(arg, ast.Call) and (
                    isinstance(arg.func, ast.Name) and arg.func.id == "_ptr"
                    or isinstance(arg.func, ast.Attribute) and arg.func.attr in ("_stream", "data_ptr", "byref"))
                assert pointer == (kind == "p"), f"{path.name}:{node.lineno}: {name}: {ast.unparse(arg)}"
            seen.add(name)
    assert len(seen) >= 30
