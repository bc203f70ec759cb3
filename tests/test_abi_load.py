"""CPU tests of the drop-in boundary: the library loads, exports every symbol
the header declares, and keeps the reference's error convention.  No compute
call needs a GPU here."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "gonngpu.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"GONNGPU_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)


def test_header_declares_the_reference_hot_path_symbols():
    names = set(declared_symbols())
    for ref_name in ["create_gpu_buffer", "retrieve_gpu_buffer_data", "release_gpu_buffer",
                     "free_c_error_message", "perform_mps_matrix_multiplication",
                     "perform_mps_matrix_transpose", "perform_mps_matrix_add_broadcast",
                     "perform_activation_relu_forward", "perform_activation_relu_backward",
                     "perform_fused_linear_activation", "perform_optimized_gemm",
                     "allocateSharedMemory", "createGPUBufferFromSharedMemory"]:
        assert ref_name in names


def test_library_exports_every_declared_symbol(built_lib):
    handle = ctypes.CDLL(built_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in gonngpu.h but not exported"
    # and the binding's signature table covers the same set
    assert set(built_lib.SIGNATURES) == set(names)


def test_header_compiles_as_plain_c(tmp_path):
    import subprocess
    src = tmp_path / "t.c"
    src.write_text('#include "gonngpu.h"\nint main(void){CError e; e.message=0; return (int)sizeof(GPUPtr)-8+(e.message!=0);}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c",
                    str(src), "-o", str(tmp_path / "t.o")], check=True)


def test_error_convention_without_touching_a_gpu(built_lib):
    g = built_lib
    lib = g.lib()
    assert lib.release_gpu_buffer(None) == 0          # NULL is a no-op, as in the reference
    lib.free_c_error_message(None)                    # must not crash
    assert b"sm_100a" in lib.gonngpu_version()
    # a handle that was never issued is rejected with the reference's code and a message
    err = g.CError()
    bogus = ctypes.c_void_p(0x1234)
    out = (ctypes.c_float * 4)()
    rc = lib.retrieve_gpu_buffer_data(bogus, out, 16, ctypes.byref(err))
    assert rc == -1 and err.message
    assert b"Invalid GPU buffer pointer" in ctypes.string_at(err.message)
    lib.free_c_error_message(err.message)
    # transpose checks its dimensions before anything else (-2), buffers next (-3)
    err = g.CError()
    assert lib.perform_mps_matrix_transpose(bogus, 2, 3, bogus, 2, 3, None, ctypes.byref(err)) == -2
    lib.free_c_error_message(err.message)
    err = g.CError()
    assert lib.perform_mps_matrix_transpose(bogus, 2, 3, bogus, 3, 2, None, ctypes.byref(err)) == -3
    lib.free_c_error_message(err.message)
    err = g.CError()
    assert lib.perform_mps_matrix_multiplication(bogus, 2, 3, bogus, 3, 2, bogus, 2, 2, None,
                                                 ctypes.byref(err)) == -2
    lib.free_c_error_message(err.message)
    # err may be NULL
    assert lib.perform_activation_relu_forward(bogus, 4, bogus, None, None) == -1
