"""Flagship models through the native path on one GPU: loss goes down, native kernels really ran."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(model, opt):
    from flodl_b200.parallel.engine import TrainEngine
    return TrainEngine(model, opt, max_grad_norm=1.0)


def test_resnet20_trains_and_matches_pytorch_forward():
    from flodl_b200 import nn, ops
    from flodl_b200.autograd import Variable
    from flodl_b200.models.resnet import resnet20
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    m = resnet20(10, dev)
    m.set_training(True)
    x = torch.randn(32, 3, 32, 32, device=dev)
    y = torch.randint(0, 10, (32,), device=dev)
    # fp32 forward: native BN (fused add/ReLU) vs the PyTorch ops with the same parameters
    out_native = m.forward(Variable.wrap(x)).t.detach()
    for b_ in m.buffers():
        b_.get().copy_(torch.zeros_like(b_.get()) if b_.name == "running_mean" else torch.ones_like(b_.get()))
    ops.set_native(False)
    try:
        out_ref = m.forward(Variable.wrap(x)).t.detach()
    finally:
        ops.set_native(True)
    assert (out_native - out_ref).abs().max().item() < 2e-3
    with nn.AutocastGuard(torch.bfloat16):
        eng = _engine(m, lambda ps: nn.SGD(ps, 0.05, 0.9, 1e-4))
        ops.FLAGS.count_launches, ops.FLAGS.launches = True, 0
        losses = [eng.step(lambda: nn.cross_entropy_loss(m.forward(Variable.wrap(x.bfloat16())), Variable.wrap(y))).item() for _ in range(12)]
        ops.FLAGS.count_launches = False
    assert ops.FLAGS.launches > 12 * 40          # BN fwd/bwd + CE + SGD kernels are this library's
    assert losses[-1] < losses[0] * 0.7, losses


def test_decoder_lm_trains_with_graph_replay():
    from flodl_b200 import nn
    from flodl_b200.models.gpt import DecoderLM, DecoderLMConfig
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    cfg = DecoderLMConfig(vocab_size=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, max_seq=128, dropout=0.1)
    m = DecoderLM(cfg, dev)
    m.set_training(True)
    ids = torch.randint(0, 512, (4, 129), device=dev)
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    with nn.AutocastGuard(torch.bfloat16):
        eng = _engine(m, lambda ps: nn.AdamW(ps, 3e-3, 0.0))
        first = eng.step(lambda: m.loss(x, y)).item()
        eng.capture(lambda a, b: m.loss(a, b), [x, y], warmup=2)
        for _ in range(30):
            last = eng.replay([x, y])
        torch.cuda.synchronize()
        eng.check()
    assert last.item() < first * 0.6, (first, last.item())


def test_bert_mlm_native_vs_pytorch_loss_and_grads():
    from flodl_b200 import nn, ops
    from flodl_b200.hf.models.bert import BertConfig, BertForMaskedLM, build_extended_attention_mask
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    cfg = BertConfig(vocab_size=1000, hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=256,
                     max_position_embeddings=128, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    head = BertForMaskedLM.on_device(cfg, dev)
    B, S = 4, 128
    ids = torch.randint(0, 1000, (B, S), device=dev)
    pos = torch.arange(S, device=dev).expand(B, S).contiguous()
    tt = torch.zeros(B, S, dtype=torch.long, device=dev)
    am = torch.ones(B, S, device=dev)
    am[:, 100:] = 0
    mask = build_extended_attention_mask(am)
    labels = torch.full((B, S), -100, device=dev)
    labels[:, 3::9] = ids[:, 3::9]
    named = head.graph().named_parameters()
    params = [p.t for _, p in named]

    def run():
        for p in params:
            p.grad = None
        with nn.AutocastGuard(torch.bfloat16):
            loss = head.compute_loss([ids, pos, tt, mask], labels)
        loss.backward()
        return loss.item(), [p.grad.float().clone() for p in params]

    l_native, g_native = run()
    ops.set_native(False)
    try:
        l_ref, g_ref = run()
    finally:
        ops.set_native(True)
    assert abs(l_native - l_ref) < 0.05 * max(1.0, abs(l_ref)), (l_native, l_ref)
    # the key-projection bias has a mathematically zero gradient (softmax is shift-invariant), so
    # both sides hold rounding noise there: leave it out of the direction check
    cos = {n: torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
           for (n, _), a, b in zip(named, g_native, g_ref) if b.abs().max() > 0 and not n.endswith("key.bias")}
    worst = min(cos, key=cos.get)
    assert cos[worst] > 0.98, (worst, cos[worst])


def _loss_curve(build, step_inputs, opt_factory, native: bool, steps: int = 40, torch_opt=None):
    """Losses of `steps` training steps from a fixed seed.

    native=True : the product path - bf16 autocast, this library's kernels, `TrainEngine` with its flat
                  buffers and fused optimizer.
    native=False: the yardstick - the same modules through plain PyTorch fp32 ops (`ops.set_native(False)`,
                  no autocast) and a stock `torch.optim` optimizer, nothing of the engine."""
    from flodl_b200 import nn, ops
    from flodl_b200.parallel.engine import TrainEngine
    torch.manual_seed(1234)
    ops.core.manual_seed(7)
    ops.set_native(native)
    try:
        model, loss_fn = build()
        out = []
        if native:
            with nn.AutocastGuard(torch.bfloat16):
                eng = TrainEngine(model, opt_factory)
                for i in range(steps):
                    inp = step_inputs[i % len(step_inputs)]
                    out.append(eng.step(lambda: loss_fn(*inp)).item())
        else:
            opt = torch_opt([p.t for p in model.parameters()])
            for i in range(steps):
                inp = [t.float() if t.is_floating_point() else t for t in step_inputs[i % len(step_inputs)]]
                opt.zero_grad()
                loss = loss_fn(*inp).t
                loss.backward()
                opt.step()
                out.append(loss.item())
        torch.cuda.synchronize()
        return out
    finally:
        ops.set_native(True)


def _assert_parity(a, b, what, step_tol=0.10, tail_tol=0.05):
    """The bf16 product path against fp32 PyTorch: the curves must track each other all the way (no
    drift that compounds), and both must have learned."""
    assert a[-1] < 0.8 * a[0] and b[-1] < 0.8 * b[0], (what, a[0], a[-1], b[0], b[-1])
    worst = max(abs(x - y) / max(abs(y), 0.05) for x, y in zip(a, b))
    assert worst < step_tol, (what, worst, a[-5:], b[-5:])
    tail = abs(sum(a[-10:]) - sum(b[-10:])) / abs(sum(b[-10:]))
    assert tail < tail_tol, (what, tail)


def test_training_loss_parity_native_vs_pytorch_ops_bert_tiny():
    from flodl_b200 import nn
    from flodl_b200.hf.models.bert import BertConfig, BertForMaskedLM, build_extended_attention_mask
    dev = torch.device("cuda", 0)
    cfg = BertConfig(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=256,
                     max_position_embeddings=128, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    B, S = 8, 128
    g = torch.Generator().manual_seed(3)
    batches = []
    for _ in range(4):
        ids = torch.randint(0, 512, (B, S), generator=g)
        labels = torch.full((B, S), -100, dtype=torch.long)
        m = torch.rand(B, S, generator=g) < 0.15
        labels[m] = ids[m]
        batches.append((ids.to(dev), torch.arange(S, device=dev).expand(B, S).contiguous(), torch.zeros(B, S, dtype=torch.long, device=dev),
                        build_extended_attention_mask(torch.ones(B, S, device=dev)), labels.to(dev)))

    def build():
        head = BertForMaskedLM.on_device(cfg, dev)
        head.graph().set_training(True)
        return head.graph(), lambda ids, pos, tt, am, lab: head.compute_loss([ids, pos, tt, am], lab)
    a = _loss_curve(build, batches, lambda ps: nn.AdamW(ps, 2e-3, 0.01), True, 32)
    b = _loss_curve(build, batches, None, False, 32, lambda ps: torch.optim.AdamW(ps, lr=2e-3, weight_decay=0.01))
    _assert_parity(a, b, "bert-tiny")


def test_training_loss_parity_native_vs_pytorch_ops_decoder_lm():
    from flodl_b200 import nn
    from flodl_b200.models.gpt import DecoderLM, DecoderLMConfig
    dev = torch.device("cuda", 0)
    cfg = DecoderLMConfig(vocab_size=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, max_seq=128, dropout=0.0)
    g = torch.Generator().manual_seed(4)
    base = torch.randint(0, 512, (96,), generator=g)
    stream = base.repeat(64)
    batches = []
    for i in range(4):
        ids = torch.stack([stream[j * 31 + i:j * 31 + i + 129] for j in range(8)]).to(dev)
        batches.append((ids[:, :-1].contiguous(), ids[:, 1:].contiguous()))

    def build():
        m = DecoderLM(cfg, dev)
        m.set_training(True)
        return m, lambda x, y: m.loss(x, y)
    a = _loss_curve(build, batches, lambda ps: nn.AdamW(ps, 2e-3, 0.0), True, 32)
    b = _loss_curve(build, batches, None, False, 32, lambda ps: torch.optim.AdamW(ps, lr=2e-3, weight_decay=0.0))
    _assert_parity(a, b, "decoder-lm", step_tol=0.15, tail_tol=0.08)


def test_training_loss_parity_native_vs_pytorch_ops_resnet20():
    from flodl_b200 import nn
    from flodl_b200.autograd import Variable
    from flodl_b200.models.resnet import resnet20
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(64, 3, 32, 32, generator=g)
    y = (x.mean((1, 2, 3)) * 40).long().clamp(-4, 5) + 4         # a learnable labelling of the images
    batches = [(x.to(dev).bfloat16(), y.to(dev))]

    def build():
        m = resnet20(10, dev)
        m.set_training(True)
        return m, lambda a, b: nn.cross_entropy_loss(m.forward(Variable.wrap(a)), Variable.wrap(b))
    a = _loss_curve(build, batches, lambda ps: nn.SGD(ps, 0.05, 0.9, 1e-4), True, 30)
    b = _loss_curve(build, batches, None, False, 30, lambda ps: torch.optim.SGD(ps, lr=0.05, momentum=0.9, weight_decay=1e-4))
    # one batch is memorised within a dozen steps: compare the descent itself, then the (tiny) end values
    assert a[-1] < 0.1 * a[0] and b[-1] < 0.1 * b[0], (a[0], a[-1], b[0], b[-1])
    assert abs(sum(a[:10]) - sum(b[:10])) / abs(sum(b[:10])) < 0.15, (a[:10], b[:10])
    assert abs(a[-1] - b[-1]) < 0.05, (a[-1], b[-1])


@pytest.mark.parametrize("opt_name", ["RMSprop", "Adagrad", "RAdam", "NAdam"])
def test_bf16_weight_copy_follows_every_optimizer(opt_name):
    """The forward GEMMs read a bf16 copy of the parameters. Only Adam / AdamW / SGD refresh it inside their fused
    kernel; every other optimizer must leave it equal to the updated fp32 values too, or training would keep using the
    initial weights."""
    from flodl_b200 import nn
    from flodl_b200.models.gpt import DecoderLM, DecoderLMConfig
    from flodl_b200.parallel.engine import TrainEngine
    torch.manual_seed(0)
    cfg = DecoderLMConfig(vocab_size=128, d_model=64, n_layers=1, n_heads=1, d_ff=128, max_seq=32, dropout=0.0)
    model = DecoderLM(cfg, "cuda")
    model.set_training(True)
    ids = torch.randint(0, 128, (4, 33), device="cuda")
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    with nn.AutocastGuard(torch.bfloat16):
        eng = TrainEngine(model, lambda ps: getattr(nn, opt_name)(ps, 1e-2))
        before = eng.flat.params.clone()
        losses = [float(eng.step(lambda: model.loss(x, y))) for _ in range(6)]
    torch.cuda.synchronize()
    assert not torch.equal(eng.flat.params, before)
    assert torch.equal(eng.flat.shadow, eng.flat.params.to(torch.bfloat16)), "the bf16 copy was not refreshed after the step"
    assert losses[-1] < losses[0]
