"""The local MPI subset used to build the reference baseline (``baseline/shims``): point-to-point with wildcards from
several threads, collectives, non-blocking receive.  The launcher must also stop the other ranks when one fails."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIMS = os.path.join(ROOT, "baseline", "shims")


@pytest.fixture(scope="module")
def selftest(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("mpishim") / "selftest")
    subprocess.run(["g++", "-std=c++17", "-O2", "-pthread", "-I", SHIMS, os.path.join(SHIMS, "tests", "selftest.cc"),
                    os.path.join(SHIMS, "mpi_shim.cc"), "-o", exe], check=True)
    return exe


@pytest.mark.parametrize("ranks", [1, 2, 4, 5])
def test_point_to_point_and_collectives(selftest, ranks):
    r = subprocess.run([sys.executable, os.path.join(SHIMS, "mpirun_local.py"), "-np", str(ranks), "--timeout", "120", selftest],
                       capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stderr[-2000:]
    assert f"selftest ok on {ranks} ranks" in r.stdout


def test_launcher_stops_the_job_when_a_rank_fails(tmp_path):
    src = tmp_path / "fail.cc"
    src.write_text('#include "mpi.h"\n#include <stdlib.h>\nint main(int c, char** v) { int p; MPI_Init_thread(&c, &v, 3, &p); int r;\n'
                   'MPI_Comm_rank(0, &r); if (r == 1) exit(3); int x; MPI_Status s; MPI_Recv(&x, 1, MPI_INT, 1, 5, 0, &s); return 0; }\n')
    exe = str(tmp_path / "fail")
    subprocess.run(["g++", "-std=c++17", "-pthread", "-I", SHIMS, str(src), os.path.join(SHIMS, "mpi_shim.cc"), "-o", exe], check=True)
    sys.path.insert(0, SHIMS)
    import mpirun_local
    code, _ = mpirun_local.launch(3, [exe], timeout=60)
    assert code == 3          # rank 1's exit code; ranks 0 and 2 were blocked in MPI_Recv / the final barrier and got terminated
