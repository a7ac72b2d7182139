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
