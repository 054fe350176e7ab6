"""Failure detection on the host, with gloo ranks on the CPU: a rank that never joins, a rank that leaves between
steps, and a collective whose peer does not take part.  No GPU is involved and nothing hangs: every wait has a limit."""
import os
import socket
import subprocess
import sys
import textwrap

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn(code: str, rank: int, world: int, port: int):
    env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
               OMP_NUM_THREADS="1", PYTHONPATH=ROOT)
    return subprocess.Popen([sys.executable, "-c", textwrap.dedent(code)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)


def test_a_rank_that_never_joins_surfaces_as_an_exception():
    code = """
        from onnxruntime_b200.parallel.dist import init_distributed
        try:
            init_distributed("gloo", timeout_s=3)
            print("JOINED")
        except Exception as e:
            print("BOOTSTRAP-FAILED", type(e).__name__)
    """
    p = _spawn(code, 0, 2, _free_port())   # rank 1 is never started
    out, _ = p.communicate(timeout=120)
    assert "BOOTSTRAP-FAILED" in out and "JOINED" not in out, out


STEP = """
    import numpy as np, sys, time
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    from onnxruntime_b200.parallel.dist import init_distributed, RankMonitor, RankLeft
    info = init_distributed("gloo", timeout_s={timeout})
    T = ol.TensorProto
    g = ol.make_graph([ol.make_node("AllReduce", ["x"], ["y"], domain="com.microsoft")], "g",
                      [ol.make_tensor_value_info("x", T.FLOAT, [4])], [ol.make_tensor_value_info("y", T.FLOAT, [4])])
    sess = ort.InferenceSession(ol.make_model(g).serialize(), providers=["CPUExecutionProvider"], dist=info)
    mon = RankMonitor(info.rank, info.world_size)
    x = np.full(4, info.rank + 1, np.float32)
"""


def test_a_rank_that_leaves_between_steps_is_noticed_before_the_next_launch():
    code = STEP.format(timeout=30) + """
    for step in range(5):
        try:
            mon.check()
        except RankLeft as e:
            print("NOTICED at step", step, e)
            break
        y = sess.run(None, {"x": x})[0]
        assert float(y[0]) == 3.0
        if info.rank == 1 and step == 1:
            mon.leave("maintenance")          # between steps: nothing of this rank is in flight
            print("LEFT after step", step)
            break
        time.sleep(0.3)                        # the other rank's announcement has time to land
    """
    port = _free_port()
    procs = [_spawn(code, r, 2, port) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert "LEFT after step 1" in outs[1], outs[1]
    assert "NOTICED at step 2" in outs[0] and "maintenance" in outs[0], outs[0]


def test_a_collective_whose_peer_stays_away_times_out_with_an_error():
    code = STEP.format(timeout=4) + """
    if info.rank == 0:
        try:
            sess.run(None, {"x": x})
            print("NO-ERROR")
        except Exception as e:
            print("COLLECTIVE-FAILED", type(e).__name__)
    else:
        time.sleep(12)   # takes no part in the collective and only leaves once rank 0 has given up
    """
    port = _free_port()
    procs = [_spawn(code, r, 2, port) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert "COLLECTIVE-FAILED" in outs[0] and "NO-ERROR" not in outs[0], outs[0]
