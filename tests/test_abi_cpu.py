"""The C-ABI library builds for sm_100a, loads without a GPU, and exports exactly the entry
points include/llm_cuda.h declares. No compute call is made here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "llm_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(llm_cuda_[a-z_]+)\s*\(", text)))


def test_header_and_library_agree_on_the_exported_symbols():
    from scriptonait_b200 import native
    lib = native.load()
    declared = _declared_functions()
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in llm_cuda.h but not exported"
    assert sorted(native.EXPORTS) == declared


def test_struct_layout_matches_the_header(tmp_path):
    """sizeof/offsetof of the two ABI structs as the C compiler sees them."""
    import subprocess
    from scriptonait_b200 import native
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "llm_cuda.h"\n'
                   'int main(void){printf("%zu %zu %zu %zu %zu %zu\\n", sizeof(llm_cuda_sample_args),'
                   'offsetof(llm_cuda_sample_args, tokens), offsetof(llm_cuda_sample_args, stream),'
                   'offsetof(llm_cuda_sample_args, history), sizeof(llm_cuda_sampling_config),'
                   'offsetof(llm_cuda_sampling_config, allowed));return 0;}\n')
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    A, S = native.SampleArgs, native.SamplingConfigC
    assert got == [ctypes.sizeof(A), A.tokens.offset, A.stream.offset, A.history.offset, ctypes.sizeof(S), S.allowed.offset]


def test_abi_version_and_defaults_without_a_gpu():
    from scriptonait_b200 import native
    lib = native.load()
    assert lib.llm_cuda_abi_version() == native.ABI_VERSION
    c = native.SamplingConfigC()
    lib.llm_cuda_sampling_config_default(ctypes.byref(c))
    assert (round(c.temperature, 6), c.top_k, round(c.top_p, 6), c.min_p, round(c.repetition_penalty, 6),
            c.repetition_window, c.seed) == (0.9, 40, 0.95, 0.0, 1.1, 128, 0)


def test_no_device_is_an_error_not_a_fallback():
    """Without a GPU, creating a sampler must fail loudly; nothing computes on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import scriptonait_b200 as sb
    with pytest.raises(sb.LlmCudaError) as e:
        sb.Sampler()
    assert e.value.code == sb.native.ERR_NO_DEVICE
    assert "no CPU path" in str(e.value)


def test_product_package_never_touches_the_oracle():
    pkg = os.path.join(ROOT, "scriptonait_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text and "liboracle" not in text, f


def test_cpp_header_compiles_against_the_library(tmp_path):
    """include/llm_cuda.hpp is a header-only C++ layer over the C ABI: it must compile with g++ and
    link against libllm_cuda.so (the GPU suite also runs the program)."""
    import subprocess
    from scriptonait_b200 import native
    native.load()
    src = tmp_path / "hpp_link.cpp"
    src.write_text('#include "llm_cuda.hpp"\n'
                   'int main(int argc, char**) {\n'
                   '    llm_cuda::SamplingConfig cfg;\n'
                   '    auto rng = llm_cuda::Rng::seed_from_u64(1234);\n'
                   '    if (argc > 100) { llm_cuda::Sampler s; return (int)s.sample({1.f, 2.f}, cfg.temperature, rng); }\n'
                   '    return (rng.next_u64() == 0xbb0cf61b2f181cdbull && cfg.top_k == 40) ? 0 : 1;\n'
                   '}\n')
    exe = tmp_path / "hpp_link"
    libdir = os.path.dirname(native.library_path())
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", libdir, "-lllm_cuda", f"-Wl,-rpath,{libdir}"], check=True)
    assert subprocess.run([str(exe)]).returncode == 0  # SplitMix64's first output for seed 1234 (rng.rs:16-22)


def test_static_entry_point_rejects_bad_arguments_before_touching_a_device():
    """The allocation-free entry point makes the handle-based entry point's argument checks: a logits
    pointer that is not element aligned, a NaN penalty or an impossible history come back as
    LLM_CUDA_ERR_BAD_ARGUMENT, with nothing launched (this runs without a GPU)."""
    from scriptonait_b200 import native as N
    lib = N.load()
    tokens = (ctypes.c_uint32 * 4)()

    def args(**kw):
        a = N.SampleArgs()
        a.struct_size = ctypes.sizeof(N.SampleArgs)
        a.logits_dtype = N.DTYPE_F32
        a.logits = 0x10000
        a.batch, a.vocab, a.row_stride_elems = 4, 1000, 1000
        a.temperature, a.top_k, a.top_p, a.repetition_penalty = 1.0, 8, 1.0, 1.0
        a.tokens = ctypes.addressof(tokens)
        for k, v in kw.items():
            setattr(a, k, v)
        return a

    for bad, text in [(args(logits=0x10002), b"aligned"), (args(logits=0x10001, logits_dtype=N.DTYPE_BF16), b"aligned"),
                      (args(repetition_penalty=float("nan")), b"NaN"), (args(temperature=float("nan")), b"NaN"),
                      (args(history=0x20000, history_stride=4, history_len=9), b"history_len"),
                      (args(row_stride_elems=10), b"row_stride"), (args(struct_size=8), b"struct_size"),
                      (args(logits_dtype=7), b"dtype"), (args(vocab=0), b"vocab")]:
        assert lib.llm_cuda_sample_batch_static(0, ctypes.byref(bad)) == N.ERR_BAD_ARGUMENT
        assert text in lib.llm_cuda_static_last_error(), lib.llm_cuda_static_last_error()
