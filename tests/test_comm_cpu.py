"""Host-side failure handling of the gradient-exchange entry points (he_comm_*), without a GPU and
without NCCL: the library is pointed at a stand-in libnccl (tests/fake_nccl.c) whose communicator never
becomes ready, or reports an asynchronous error, or works.  Each scenario runs in a child process because
the library binds its NCCL once per process."""
import os
import subprocess
import sys
import textwrap

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_nccl") / "libfake_nccl.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(out), os.path.join(HERE, "fake_nccl.c")], check=True)
    return str(out)


def _child(fake, mode, body):
    code = textwrap.dedent("""
        import ctypes as C, sys, time
        sys.path.insert(0, %r)
        from helium_b200._lib import lib
        fake = C.CDLL(%r)
        err = lambda: lib.he_last_error_string().decode()
        uid = C.create_string_buffer(128)
        assert lib.he_comm_unique_id(uid) == 0, err()
        comm = C.c_void_p()
    """ % (ROOT, fake)) + textwrap.dedent(body)
    env = dict(os.environ, HE_NCCL_LIBRARY=fake, FAKE_NCCL_MODE=mode)
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_a_rank_that_never_joins_ends_in_deadline_and_abort(fake_nccl):
    out = _child(fake_nccl, "never_joins", """
        t0 = time.perf_counter()
        rc = lib.he_comm_create(None, 0, 2, uid, 0, 300, C.byref(comm))
        dt = time.perf_counter() - t0
        assert rc == -7, (rc, err())                      # HE_ERR_COMM_TIMEOUT
        assert 0.25 < dt < 5.0, dt                        # the 300 ms deadline, not a hang
        assert not comm.value
        assert fake.fake_nccl_abort_count() == 1          # the half-made communicator was aborted
        assert "never joined" in err() and "aborted" in err(), err()
        print("ok")
    """)
    assert "ok" in out


def test_an_asynchronous_nccl_error_aborts_the_communicator(fake_nccl):
    out = _child(fake_nccl, "async_error", """
        rc = lib.he_comm_create(None, 1, 2, uid, 0, 300, C.byref(comm))
        assert rc == -6, (rc, err())                      # HE_ERR_COMM
        assert "remote process exited" in err(), err()
        assert fake.fake_nccl_abort_count() == 1
        print("ok")
    """)
    assert "ok" in out


def test_argument_checks_come_before_any_collective(fake_nccl):
    out = _child(fake_nccl, "ok", """
        assert lib.he_comm_create(None, 2, 2, uid, 0, 300, C.byref(comm)) == -1       # rank out of range
        assert lib.he_comm_create(None, 0, 1, uid, 8, 300, C.byref(comm)) == 0, err()
        r, w, m = C.c_int32(), C.c_int32(), C.c_int32()
        assert lib.he_comm_info(comm, C.byref(r), C.byref(w), C.byref(m)) == 0 and (r.value, w.value, m.value) == (0, 1, 8)
        bufs = (C.c_void_p * 2)(0x1000, 0x2000)
        counts = (C.c_size_t * 2)(16, 0)
        assert lib.he_allreduce_grads(comm, bufs, counts, 2, 2, 1, None) == -1 and "0 elements" in err()   # empty buffer
        counts[1] = 8
        assert lib.he_allreduce_grads(comm, bufs, counts, 2, 4, 1, None) == -1 and "f16, bf16 or f32" in err()   # bool gradients
        bufs[1] = None
        assert lib.he_allreduce_grads(comm, bufs, counts, 2, 2, 1, None) == -1 and "null" in err()
        assert fake.fake_nccl_allreduce_count() == 0      # nothing reached NCCL
        bufs[1] = 0x2000
        assert lib.he_allreduce_grads(comm, bufs, counts, 2, 2, 1, None) == 0, err()
        assert fake.fake_nccl_allreduce_count() == 2      # one group of two collectives
        assert lib.he_comm_poll(comm) == 0
        assert lib.he_comm_abort(comm) == 0 and fake.fake_nccl_abort_count() == 1
        assert lib.he_comm_poll(comm) == -6               # aborted communicators stay unusable
        assert lib.he_allreduce_grads(comm, bufs, counts, 2, 2, 1, None) == -6
        lib.he_comm_destroy(comm)
        assert fake.fake_nccl_destroy_count() == 0        # an aborted communicator is not destroyed twice
        print("ok")
    """)
    assert "ok" in out


def test_missing_nccl_is_reported_not_crashed():
    code = ("import ctypes as C, sys; sys.path.insert(0, %r); from helium_b200._lib import lib; "
            "uid = C.create_string_buffer(128); rc = lib.he_comm_unique_id(uid); "
            "assert rc == -6, rc; assert b'could not load NCCL' in lib.he_last_error_string(); print('ok')" % ROOT)
    r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, HE_NCCL_LIBRARY="/nonexistent/libnccl.so.2"),
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
