"""Runs the native (C / C++) test programs that need no GPU.  Exit code 77 means skipped, as in
the reference's CTest setup."""
import subprocess
from pathlib import Path

import pytest

TESTS = Path(__file__).resolve().parent.parent / "nano_nccl_b200" / "lib" / "tests"
CPU_PROGRAMS = ["bootstrap_test", "c_api", "simple_protocol_test", "socket_protocol_test", "host_ring_test",
                "rdma_protocol_test", "rdma_proxy_test", "rdma_timeline_test", "rdma_endpoint_test", "topology_tuner_test",
                "ring_turnaround_test", "rdma_ibv_contract_test"]


@pytest.mark.parametrize("name", CPU_PROGRAMS)
def test_native_program(name, native_build):
    exe = TESTS / name
    assert exe.exists(), f"{exe} was not built"
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    if proc.returncode == 77:
        pytest.skip(proc.stdout + proc.stderr)
    assert proc.returncode == 0, proc.stdout + proc.stderr


@pytest.mark.parametrize("nranks", [1, 2, 4, 5])
def test_minimal_mpi_under_the_launcher(nranks, native_build):
    """Every MPI entry point the library uses, as separate processes started by the bundled launcher."""
    import subprocess

    lib = TESTS.parent
    p = subprocess.run([str(lib / "nano_nccl_mpirun"), "-np", str(nranks), "--timeout", "60", str(TESTS / "minimpi_check")],
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and f"minimpi_check ok ({nranks} ranks)" in p.stdout, p.stdout + p.stderr


def test_launcher_reports_a_failing_rank(native_build):
    """A rank that exits non-zero makes the launcher exit non-zero (and it does not wait for the time limit)."""
    import subprocess
    import time

    lib = TESTS.parent
    t0 = time.time()
    p = subprocess.run([str(lib / "nano_nccl_mpirun"), "-np", "2", "--timeout", "60", "/bin/sh", "-c",
                        'test "$OMPI_COMM_WORLD_RANK" = 0'], capture_output=True, text=True, timeout=120)
    assert p.returncode != 0
    assert time.time() - t0 < 30


def test_mpi_c_abi_fails_cleanly_without_a_gpu(native_build):
    """Creating a communicator through the MPI C ABI on a machine without GPUs: a diagnostic on every rank,
    no hang, a second attempt possible."""
    import subprocess

    lib = TESTS.parent
    p = subprocess.run([str(lib / "nano_nccl_mpirun"), "-np", "2", "--timeout", "60", str(TESTS / "mpi_c_api_nogpu")],
                       capture_output=True, text=True, timeout=120)
    if p.returncode == 77:
        pytest.skip("GPUs are present: the GPU suites cover communicator creation")
    assert p.returncode == 0 and "mpi_c_api_nogpu ok" in p.stdout, p.stdout + p.stderr
    assert "device selection failed" in p.stdout


def test_launcher_time_limit_ends_hanging_ranks(native_build):
    """Ranks that never finish are ended by the launcher's own time limit (it signals the processes it started)."""
    import subprocess
    import time

    lib = TESTS.parent
    t0 = time.time()
    p = subprocess.run([str(lib / "nano_nccl_mpirun"), "-np", "2", "--timeout", "2", "/bin/sleep", "100"],
                       capture_output=True, text=True, timeout=60)
    assert p.returncode != 0
    assert time.time() - t0 < 20, "the launcher did not enforce its limit"


def test_install_tree_serves_a_c_program_under_the_reference_library_name(native_build, tmp_path):
    """`_build.install(prefix)` lays out include/, lib/ and a CMake package; a plain C program compiled against the
    installed headers and linked only with -lnano_nccl_mpi_c (the reference's shared library name) runs."""
    import subprocess

    where = native_build.install(tmp_path / "prefix")
    assert (where["include"] / "nano_nccl.h").exists() and (where["include"] / "mpi_c_api.h").exists()
    assert (where["lib"] / "libnano_nccl.so").exists() and (where["lib"] / "libnano_nccl_mpi_c.so").exists()
    assert "nano_nccl::nano_nccl_mpi_c" in (where["cmake"] / "nano_ncclConfig.cmake").read_text()
    src = tmp_path / "abi.c"
    src.write_text('#include <nano_nccl/nano_nccl.h>\n#include <stdio.h>\n'
                   'int main(void) {\n'
                   '    if (nano_nccl_abi_version() != NANO_NCCL_ABI_VERSION) return 1;\n'
                   '    if (nano_nccl_destroy_communicator(NULL) != NANO_NCCL_STATUS_SUCCESS) return 2;\n'
                   '    printf("abi %u via the alias\\n", nano_nccl_abi_version());\n    return 0;\n}\n')
    exe = tmp_path / "abi"
    cuda_inc = str(native_build.CUDA_HOME / "include")
    subprocess.run(["gcc", "-std=c11", "-I", str(tmp_path / "prefix" / "include"), "-I", cuda_inc, str(src), "-o", str(exe),
                    "-L", str(where["lib"]), "-lnano_nccl_mpi_c", "-Wl,-rpath," + str(where["lib"]),
                    "-Wl,-rpath-link," + str(where["lib"])], check=True, capture_output=True, text=True)
    p = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert p.returncode == 0 and "abi 2 via the alias" in p.stdout, p.stdout + p.stderr
