"""Load-stage timers and the opt-in tensor-parallel host timeline."""
import io

from rexl3_b200.utils import loadstats, trace


def test_loadstats_accumulate_and_render():
    loadstats.reset()
    with loadstats.stage("pack", "read", 1000):
        pass
    loadstats.add("pack", "read", 0.5, 24)
    loadstats.add("model", "upload", 1.25, 7)
    snap = loadstats.snapshot()
    assert snap[("pack", "read")][1:] == (1024, 2) and snap[("pack", "read")][0] >= 0.5
    text = loadstats.render()
    assert 'rexl3_load_stage_bytes{component="pack",stage="read"} 1024' in text
    assert 'rexl3_load_stage_seconds{component="model",stage="upload"} 1.25' in text
    assert 'rexl3_load_stage_calls{component="pack",stage="read"} 2' in text
    loadstats.reset()
    assert loadstats.render() == ""


def test_pack_load_fills_the_stage_timers(tmp_path):
    import dataclasses

    from rexl3_b200.models import dense
    from rexl3_b200.quant import quantize
    cfg = dataclasses.replace(dense.CONFIGS["tiny-llama"], n_layers=1, vocab=256, ffn=128)
    folder = str(tmp_path / "p")
    quantize.write_pack(folder, dense.random_weights(cfg, seed=3))
    loadstats.reset()
    quantize.load_pack(folder)
    snap = loadstats.snapshot()
    assert snap[("pack", "read")][1] > 0 and snap[("pack", "assemble")][2] == 1


def test_tp_trace_lines_and_off_by_default():
    assert not trace.TP_TRACE and not trace.NVTX
    trace.tp_event("L", 0, "ignored", 1)          # off: nothing is queued, nothing is started
    assert trace._q is None
    buf = io.StringIO()
    try:
        trace.enable_tp_trace(buf)
        trace.tp_event("L", 0, "send_op1", 64)
        trace.tp_event("F", 3, "recv_op1", 64)
        trace.flush_tp_trace()
        lines = buf.getvalue().splitlines()
        assert len(lines) == 2
        a, b = lines[0].split(), lines[1].split()
        assert a[:2] == ["TPTRACE", "L"] and a[3:] == ["0", "send_op1", "64"] and b[1] == "F" and b[3] == "3"
        assert int(a[2]) <= int(b[2])
    finally:
        trace.TP_TRACE = False
    with trace.nvtx_range("off"):
        pass
