"""Failure paths of the communicator, made to happen on the host: libdwbnq is pointed
(DWBNQ_NCCL_LIB) at a stand-in NCCL library whose all-reduce returns an error, reports an
asynchronous error, or stalls the stream with a sleeping host function - as if a peer had
not joined - so the deadline runs out without any GPU kernel waiting for anything. Each
case runs in a child process that never imports torch (the real libnccl stays unloaded)."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, ".."))
LIB = os.path.join(ROOT, "nnabla-ext-cuda_b200", "libdwbnq.so")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
OK, ERR_NCCL, ERR_TIMEOUT = 0, 4, 5


@pytest.fixture(scope="module")
def fake_nccl():
    out_dir = os.path.join(HERE, "fake_nccl", "_build")
    os.makedirs(out_dir, exist_ok=True)
    so = os.path.join(out_dir, "libfake_nccl.so")
    subprocess.run(["gcc", "-std=c99", "-D_DEFAULT_SOURCE", "-Wall", "-Werror", "-shared", "-fPIC",
                    "-I" + os.path.join(CUDA, "include"), os.path.join(HERE, "fake_nccl", "fake_nccl.c"),
                    "-L" + os.path.join(CUDA, "lib64"), "-lcudart", "-Wl,-rpath," + os.path.join(CUDA, "lib64"),
                    "-o", so], check=True, capture_output=True, text=True)
    return so


def drive(fake, mode, timeout_ms, stall_ms=1500, what="device"):
    env = dict(os.environ, DWBNQ_NCCL_LIB=fake, FAKE_NCCL_MODE=mode, FAKE_NCCL_STALL_MS=str(stall_ms),
               LD_LIBRARY_PATH=os.path.join(CUDA, "lib64") + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    r = subprocess.run([sys.executable, os.path.join(HERE, "fake_nccl", "drive.py"), LIB, str(timeout_ms), what],
                       env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_status_codes_match_the_header(dwlib):
    assert (dwlib.OK, dwlib.ERR_NCCL, dwlib.ERR_TIMEOUT) == (OK, ERR_NCCL, ERR_TIMEOUT)


def test_healthy_all_reduce(fake_nccl):
    o = drive(fake_nccl, "ok", 500)
    assert o["get_id"] == OK and o["create"] == OK and o["allreduce"] == OK and o["second_call"] == OK
    assert o["aborts"] == 0 and o["allreduces"] == 2 and o["destroy"] == OK


def test_all_reduce_error_code_is_reported(fake_nccl):
    o = drive(fake_nccl, "error", 500)
    assert o["allreduce"] == ERR_NCCL and "ncclAllReduce" in o["message"]
    assert o["aborts"] == 0


def test_deadline_aborts_the_communicator(fake_nccl):
    o = drive(fake_nccl, "stall", 300, stall_ms=1500)
    assert o["allreduce"] == ERR_TIMEOUT, o
    assert 0.25 <= o["seconds"] < 1.2, o          # gave up at the deadline, not when the stall ended
    assert "aborted" in o["message"] and o["aborts"] == 1
    # the communicator is unusable afterwards and says so, without calling into NCCL again
    assert o["second_call"] == ERR_NCCL and "aborted" in o["second_message"]
    assert o["allreduces"] == 1 and o["destroy"] == OK


def test_asynchronous_error_ends_the_wait(fake_nccl):
    o = drive(fake_nccl, "async", 5000, stall_ms=800)
    assert o["allreduce"] == ERR_NCCL and "asynchronous" in o["message"], o
    assert o["seconds"] < 0.7, o                   # reported at once, neither deadline nor stall awaited


def test_operator_call_honours_the_communicator_deadline(fake_nccl):
    """dwbnq_minmaxq_fwd with a communicator whose peer never joins (the stand-in stalls the
    stream with a sleeping host function): the deadline set on the communicator ends the
    call with a time-out and an aborted communicator."""
    o = drive(fake_nccl, "stall", 300, stall_ms=1500, what="minmaxq")
    assert o["set_deadline"] == OK
    assert o["call"] == ERR_TIMEOUT, o
    assert 0.25 <= o["seconds"] < 1.2, o
    assert "aborted" in o["message"] and o["aborts"] == 1 and o["allreduces_after_call"] == 1
    assert o["second_call"] == ERR_NCCL and "aborted" in o["second_message"]
    assert o["allreduces"] == 1 and o["destroy"] == OK


def test_operator_call_without_deadline_only_enqueues(fake_nccl):
    o = drive(fake_nccl, "stall", 0, stall_ms=300, what="minmaxq")
    assert o["call"] == OK and o["seconds"] < 0.25 and o["aborts"] == 0, o


def test_asynchronous_error_reaches_the_operator_call(fake_nccl):
    o = drive(fake_nccl, "async", 5000, stall_ms=800, what="minmaxq")
    assert o["call"] == ERR_NCCL and "asynchronous" in o["message"] and o["seconds"] < 0.7, o


def test_empty_shard_still_joins_the_all_reduce(fake_nccl):
    """A rank whose slice of the batch is empty (fewer images than ranks) must issue the
    min/max all-reduce like its peers; without a communicator the empty batch is a no-op."""
    o = drive(fake_nccl, "ok", 0, what="fused_empty")
    assert o["call"] == OK, o
    assert o["allreduces_after_call"] == 1 and o["no_comm"] == OK and o["allreduces_no_comm"] == 1
    assert o["aborts"] == 0 and o["destroy"] == OK
