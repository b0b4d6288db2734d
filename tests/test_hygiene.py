"""Rules of the code base that a reader cannot see from one file: the product
path imports no library model code, no tracing compiler and no library
attention; sources compile for sm_100a only; nothing committed reads working
files.  Checked on the text of the sources (no GPU)."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PACKAGE = ROOT / "alofa_b200"

FORBIDDEN_IMPORTS = ("transformers", "vllm", "flash_attn", "flashinfer", "triton", "tilelang", "cutlass", "xformers", "jax")


def python_sources(folder):
    return [p for p in folder.rglob("*.py") if "_build" not in p.parts]


def test_package_imports_no_library_model_code_or_compiler():
    pattern = re.compile(r"^\s*(?:from|import)\s+(" + "|".join(FORBIDDEN_IMPORTS) + r")\b", re.M)
    for path in python_sources(PACKAGE) + [ROOT / "bench.py", ROOT / "__graft_entry__.py", ROOT / "bin" / "trace_run", ROOT / "bin" / "generate"]:
        found = pattern.findall(path.read_text())
        assert not found, f"{path.relative_to(ROOT)} imports {found}"
    for path in python_sources(PACKAGE):
        text = path.read_text()
        assert "torch.compile" not in text, path
        assert "scaled_dot_product_attention" not in text, path


def test_package_shares_no_code_with_the_tests():
    """The plain implementation and the other test helpers are the oracle: the
    package, the bench, the entry points and the programs under bin/ import
    nothing from tests/ (the smoke test alone reads the plain implementation,
    to compare with it)."""
    helpers = sorted(p.stem for p in (ROOT / "tests").glob("*.py") if not p.stem.startswith("test_"))
    assert "plain_qwen2" in helpers
    pattern = re.compile(r"^\s*(?:from|import)\s+(tests|" + "|".join(helpers) + r")\b", re.M)
    for path in python_sources(PACKAGE) + [ROOT / "bench.py", ROOT / "bin" / "trace_run", ROOT / "bin" / "generate"]:
        found = pattern.findall(path.read_text())
        assert not found, f"{path.relative_to(ROOT)} imports {found} from the tests"
        assert "plain_qwen2" not in path.read_text(), path


def test_model_math_of_the_package_goes_through_its_own_kernels():
    """Parts call the package's kernels; torch is there for memory, streams and
    graphs.  No part multiplies matrices or takes a softmax with torch."""
    banned = re.compile(r"torch\.(matmul|mm|bmm|einsum|softmax|nn\.functional)|F\.(linear|softmax|silu|scaled_dot)|\s@\s")
    for path in python_sources(PACKAGE / "parts") + python_sources(PACKAGE / "engine") + python_sources(PACKAGE / "sampling"):
        for number, line in enumerate(path.read_text().splitlines(), 1):
            code = line.split("#", 1)[0]
            assert not banned.search(code), f"{path.relative_to(ROOT)}:{number}: {line.strip()}"


def test_cuda_is_built_for_sm_100a_only():
    text = (PACKAGE / "csrc" / "build.py").read_text()
    assert "compute_100a" in text and "sm_100a" in text
    assert not re.search(r"sm_(?!100a)\d+", text), "another architecture in the build flags"


def test_nothing_committed_reads_working_files():
    folder = re.compile(r"""["'/]_work[/"']""")  # the working folder as a path component or a string
    for path in python_sources(PACKAGE) + python_sources(ROOT / "tests") + [ROOT / "bench.py", ROOT / "__graft_entry__.py"]:
        if path.name == "test_hygiene.py":
            continue
        assert not folder.search(path.read_text()), path


def test_kernel_waits_are_bounded():
    """Every spin on an mbarrier goes through the bounded wait of tma.cuh: no
    bare try_wait loop elsewhere."""
    kernels = PACKAGE / "csrc" / "kernels"
    for path in list(kernels.glob("*.cu")) + list(kernels.glob("*.cuh")):
        if path.name == "tma.cuh":
            continue
        text = path.read_text()
        assert "mbarrier.try_wait" not in text and "mbarrier.test_wait" not in text, path.name
    bounded = (kernels / "tma.cuh").read_text()
    assert re.search(r"mbar_wait\(.*abort", bounded), "the shared wait takes an abort flag"
