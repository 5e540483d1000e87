"""Bounded waits of the multi-GPU C ABI (sca_mgpu_*), on the CPU against a stand-in NCCL.

The failure is made on the host: tests/fakes/fake_nccl.c plays a communicator whose peers never join (or that
reports a system error). The library must come back with a status - SCA_TIMEOUT after about the limit it was given,
with the communicator aborted - and never hang. Each case runs in a child process because the NCCL library is chosen
(SCA_NCCL_LIBRARY) when it is first loaded."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FAKE_SRC = os.path.join(ROOT, "tests", "fakes", "fake_nccl.c")


def fake_library(tmp_path):
    out = os.path.join(tmp_path, "libfake_nccl.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", FAKE_SRC, "-o", out], check=True)
    return out


def run_child(tmp_path, mode, body):
    env = dict(os.environ, SCA_NCCL_LIBRARY=fake_library(str(tmp_path)), FAKE_NCCL_MODE=mode, PYTHONPATH=ROOT)
    code = textwrap.dedent("""
        import ctypes as C, time
        from scicompute_attention_b200 import _lib
        l = _lib.lib()
        ident = C.create_string_buffer(_lib.MGPU_ID_BYTES)
        assert l.sca_mgpu_unique_id(ident) == 0
        comm = C.c_void_p()
    """) + textwrap.dedent(body)
    return subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)


def test_a_peer_that_never_joins_surfaces_a_timeout_and_aborts(tmp_path):
    proc = run_child(tmp_path, "never", """
        t0 = time.time()
        rc = l.sca_mgpu_init(ident.raw, 0, 2, 400, C.byref(comm))
        took = time.time() - t0
        fake = C.CDLL(__import__("os").environ["SCA_NCCL_LIBRARY"])
        print(rc, round(took, 2), fake.fake_nccl_aborts(), l.sca_last_error().decode())
        assert rc == 500 and 0.35 <= took < 5.0 and fake.fake_nccl_aborts() == 1 and comm.value is None
    """)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "within 400 ms" in proc.stdout and "aborted" in proc.stdout


def test_an_asynchronous_nccl_error_is_reported_and_the_communicator_aborted(tmp_path):
    proc = run_child(tmp_path, "fail", """
        rc = l.sca_mgpu_init(ident.raw, 1, 2, 2000, C.byref(comm))
        fake = C.CDLL(__import__("os").environ["SCA_NCCL_LIBRARY"])
        print(rc, fake.fake_nccl_aborts(), l.sca_last_error().decode())
        assert rc == 100 and fake.fake_nccl_aborts() == 1
    """)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "unhandled system error" in proc.stdout


def test_a_healthy_communicator_initialises_and_rejects_use_after_abort(tmp_path):
    proc = run_child(tmp_path, "ok", """
        assert l.sca_mgpu_init(ident.raw, 0, 2, 1000, C.byref(comm)) == 0 and comm.value
        assert l.sca_mgpu_init(ident.raw, 2, 2, 1000, C.byref(C.c_void_p())) == 4      # rank out of range
        assert l.sca_mgpu_allgather_triples(comm, None, None, 8, None, 0) == 4          # null payload
        assert l.sca_mgpu_abort(comm) == 0
        buf = (C.c_float * 16)()
        assert l.sca_mgpu_allgather_triples(comm, buf, buf, 8, None, 0) == 4 and b"aborted" in l.sca_last_error()
        assert l.sca_mgpu_destroy(comm) == 0
        print("ok")
    """)
    assert proc.returncode == 0, proc.stdout + proc.stderr
