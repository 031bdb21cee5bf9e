"""Other model families on one B200 in bf16: their Linear / Conv1D / norm / embedding modules run on the kernels of this
library (module rewrite), the rest stays HF; a few optimizer steps must lower the loss."""
import pytest
import torch

from tests.test_model_families_cpu import _tiny

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["opt", "bert", "gptneo", "gptj", "vit", "whisper", "qwenmoe"])
def test_family_trains_in_bf16_on_the_kernels(name):
    from aicomp_b200 import Optimus_p, ops
    torch.manual_seed(0)
    model, kind = _tiny(name)
    kw = {}
    if kind == "ids":
        data = torch.randint(1, 128, (8, 32))
        labels = data.clone()
    elif kind == "pixels":
        data, labels = torch.randn(8, 3, 32, 32), torch.randint(0, 10, (8,))
    else:
        data = {"input_features": torch.randn(8, 8, 32), "decoder_input_ids": torch.randint(1, 128, (8, 8))}
        labels = torch.randint(1, 128, (8, 8))
        kw = {"input_names": ["input_features", "decoder_input_ids"]}
    def dev(t):  # floating-point inputs (pixels, audio features) in the model's dtype
        return t.cuda().to(torch.bfloat16) if t.is_floating_point() else t.cuda()
    data = {k: dev(v) for k, v in data.items()} if isinstance(data, dict) else dev(data)
    labels = labels.cuda()
    before = ops.launch_count()
    e = Optimus_p(model, num_mb=2, use_gpu=True, dtype=torch.bfloat16, **kw)
    assert e.fused_kernels
    opt = torch.optim.AdamW(e.parameters(), lr=2e-3)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        e.run(data, labels, mode="1f1b")
        opt.step()
        losses.append(sum(e.get_loss()) / 2)
    ops.check_errors()
    assert all(l == l for l in losses), losses
    assert losses[-1] < losses[0], losses
    assert ops.launch_count() > before, "no kernel of this library ran"
