"""The serving binary's app over the CUDA backends of the three model families (random-init tiny configs): one completion each."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("config,extra", [("test-hd128", ["--kv-dtype", "fp8"]), ("test-hd128", ["--kv-dtype", "int8"]), ("test-hd128", ["--kv-dtype", "q4"]), ("test-hd128-mtp", ["--spec", "mtp"]), ("test-moe", ["--spec", "self"]), ("test-mla", ["--spec", "none"]),
                                          ("test-hybrid", ["--spec", "copy"]), ("test-hybrid-gdn", ["--spec", "copy", "--state-snapshots", "--prefix-cache", "on"])])
def test_completion_over_cuda_backend(config, extra):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from starlette.testclient import TestClient
    from rexl3_b200.server.main import make_app, parser
    args = parser().parse_args(["--backend", "cuda", "--random-init", config, "--slots", "3", "--max-model-len", "512", "--prefill-chunk", "256",
                                "--kv-tokens", "2048", "--window-rows", "16"] + extra)
    app, handle = make_app(args)
    try:
        assert handle.wait_ready(120), handle.error
        with TestClient(app) as c:
            r = c.post("/v1/completions", json={"model": args.served_model_name or config, "prompt": "hello world, this is a test", "max_tokens": 6, "temperature": 0})
            assert r.status_code == 200, r.text
            doc = r.json()
            assert doc["usage"]["completion_tokens"] >= 1 and doc["choices"][0]["finish_reason"] in ("length", "stop")
            again = c.post("/v1/completions", json={"model": args.served_model_name or config, "prompt": "hello world, this is a test", "max_tokens": 6, "temperature": 0}).json()
            assert again["choices"][0]["text"] == doc["choices"][0]["text"]          # greedy decoding is reproducible (prefix cache or not)
            assert c.get("/v1/models").json()["data"][0]["boot"]["phases"]
    finally:
        handle.stop()
