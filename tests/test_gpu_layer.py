"""The layer loop on a GPU: overlapped linears (own streams, shared q/k/v factor) against
one-at-a-time quantization of the same synthetic model."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(concurrent: bool, arch: str, tech: str, offload: bool = False):
    from crb_b200 import run as crun
    from crb_b200.synth import build_synthetic_model, synthetic_calibration
    model = build_synthetic_model(arch, n_layers=2, seed=3)
    model.seqlen = 256
    loader = synthetic_calibration(model.config.vocab_size, nsamples=8, seqlen=256, seed=1)
    args = crun.default_args(low_quant_method=tech, nsamples=8, forward_batch=4, verbose=False,
                             device="cuda:0", percdamp=0.1)
    args.concurrent_linears = concurrent
    if offload:
        args.act_offload_gib = 0.0          # activations live in pinned host memory and stream through the device
    out = crun.quant_sequential(model, loader, "cuda:0", args)
    layers, _ = crun._decoder_parts(model)
    weights = {f"{i}.{n}": m.weight.data.float().cpu().clone()
               for i, layer in enumerate(layers) for n, m in crun.find_layers(layer).items()}
    return out, weights


@pytest.mark.parametrize("arch,tech", [("opt-tiny", "crb"), ("llama-tiny", "braq")])
def test_overlapped_linears_equal_sequential(arch, tech):
    out_c, w_c = _run(True, arch, tech)
    out_s, w_s = _run(False, arch, tech)
    assert w_c.keys() == w_s.keys() and len(w_c) >= 12
    for name in w_c:
        # same kernels on the same inputs: the schedule must not change a single bit
        assert torch.equal(w_c[name], w_s[name]), name
        assert len(torch.unique(w_c[name][0])) <= 3 * 4 * (w_c[name].shape[1] // 128) + 1
    for ec, es in zip(out_c["errors"], out_s["errors"]):
        assert ec == es
    assert torch.equal(out_c["final_hidden"].cpu(), out_s["final_hidden"].cpu())
    assert out_c["error_sum"] > 0


def test_host_resident_activations_equal_device_resident():
    """Activations offloaded to pinned host memory (prefetched batch by batch, written back on a side
    stream) and weights streamed one layer ahead give the very same result."""
    out_h, w_h = _run(True, "opt-tiny", "crb", offload=True)
    out_d, w_d = _run(True, "opt-tiny", "crb", offload=False)
    assert out_h["final_hidden"].device.type == "cpu" and out_d["final_hidden"].device.type == "cuda"
    for name in w_d:
        assert torch.equal(w_h[name], w_d[name]), name
    assert torch.equal(out_h["final_hidden"], out_d["final_hidden"].cpu())
    assert out_h["errors"] == out_d["errors"]
