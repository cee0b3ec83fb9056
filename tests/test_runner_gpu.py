"""Whole-network parity: a ResNet run through the low-memory operators (both policies)
against stock PyTorch autograd in fp32 on the CPU.  Convolutions run in TF32, so outputs and
gradients are compared at the convolution tolerance (rtol 2e-2 of the tensor's scale)."""
import copy

import pytest
import torch
import torchvision

pytestmark = pytest.mark.gpu


def _rel(a, ref):
    return float((a - ref).norm() / ref.norm().clamp_min(1e-12))


def _reference_step(model, x, labels):
    model = copy.deepcopy(model).cpu().train()
    out = model(x)
    loss = torch.nn.functional.cross_entropy(out, labels)
    loss.backward()
    return out.detach(), loss.detach(), {k: p.grad.clone() for k, p in model.named_parameters()}, \
        {k: b.clone() for k, b in model.named_buffers()}


class _TinyResNet(torch.nn.Module):
    """Stem + one bottleneck with a strided downsample + classifier: every operator of the
    ResNet graph, but shallow enough that TF32 rounding is not amplified by depth."""

    def __init__(self):
        super().__init__()
        nn = torch.nn
        self.conv1 = nn.Conv2d(3, 32, 7, 2, 3, bias=False)
        self.bn1 = nn.BatchNorm2d(32)
        self.relu = nn.ReLU(inplace=True)
        self.maxpool = nn.MaxPool2d(3, 2, 1)
        self.c1 = nn.Conv2d(32, 16, 1, bias=False); self.b1 = nn.BatchNorm2d(16)
        self.c2 = nn.Conv2d(16, 16, 3, 2, 1, bias=False); self.b2 = nn.BatchNorm2d(16)
        self.c3 = nn.Conv2d(16, 64, 1, bias=True); self.b3 = nn.BatchNorm2d(64)
        self.ds = nn.Conv2d(32, 64, 1, 2, bias=False); self.bds = nn.BatchNorm2d(64)
        self.avgpool = nn.AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Linear(64, 10)

    def forward(self, x):
        x = self.maxpool(self.relu(self.bn1(self.conv1(x))))
        idt = self.bds(self.ds(x))
        out = self.relu(self.b1(self.c1(x)))
        out = self.relu(self.b2(self.c2(out)))
        out = self.b3(self.c3(out))
        out = out + idt
        out = self.relu(out)
        return self.fc(torch.flatten(self.avgpool(out), 1))


def _run_ours(model, x, labels, policy, cuda):
    from monet_b200 import runner
    from monet_b200.lm_ops.softmax import SoftmaxCrossEntropy
    gm = copy.deepcopy(model).to(cuda).train()
    r = runner.Runner(gm, getattr(runner, policy))
    out = r.forward(x.to(cuda))
    ce = SoftmaxCrossEntropy()
    loss = ce.forward(out, labels.to(cuda))
    r.backward(ce.backward())
    torch.cuda.synchronize()
    return gm, out, loss


def _torch_tf32_grads(model, x, labels, cuda):
    """Stock PyTorch on the GPU with TF32 cuDNN convolutions: the yardstick for how far TF32
    arithmetic alone moves each gradient away from the fp32 CPU reference."""
    torch.backends.cudnn.allow_tf32 = True
    try:
        tm = copy.deepcopy(model).to(cuda).train()
        torch.nn.functional.cross_entropy(tm(x.to(cuda)), labels.to(cuda)).backward()
        return {k: p.grad.detach().cpu() for k, p in tm.named_parameters()}
    finally:
        torch.backends.cudnn.allow_tf32 = False


@pytest.mark.parametrize("arch,batch", [("tiny", 16), ("resnet18", 8), ("resnet50", 8)])
def test_network_step_tracks_autograd(cuda, arch, batch):
    """Forward, loss and every parameter gradient of a whole training step through the
    operators, for both policies.  Batch-norm makes weight gradients ill-conditioned (they
    are what is left after projecting the mean and the normalised activation out), so TF32
    rounding moves them by several per cent even in stock PyTorch; the bar is therefore
    relative: no worse than 1.6x the error of PyTorch's own TF32 path, plus 2 %."""
    torch.manual_seed(0)
    model = (_TinyResNet() if arch == "tiny" else getattr(torchvision.models, arch)(num_classes=10)).train()
    x = torch.randn(batch, 3, 64, 64)
    labels = torch.randint(0, 10, (batch,))
    ref_out, ref_loss, ref_grads, ref_bufs = _reference_step(model, x, labels)
    tf32 = _torch_tf32_grads(model, x, labels, cuda)
    results = {}
    for policy in ("store_all", "low_memory"):
        gm, out, loss = _run_ours(model, x, labels, policy, cuda)
        assert _rel(out.cpu(), ref_out) < 5e-2
        assert abs(float(loss) - float(ref_loss)) < 2e-2 * max(1.0, abs(float(ref_loss)))
        for k, p in gm.named_parameters():
            assert p.grad is not None, k
            ours, theirs = _rel(p.grad.cpu(), ref_grads[k]), _rel(tf32[k], ref_grads[k])
            assert ours < 1.6 * theirs + 2e-2, (policy, k, ours, theirs)
        if arch == "tiny":
            for k, b in gm.named_buffers():
                if "num_batches" not in k:
                    assert _rel(b.cpu(), ref_bufs[k]) < 1e-2, k
        results[policy] = {k: p.grad.clone() for k, p in gm.named_parameters()}
    # the two policies run the same arithmetic apart from the batch-norm backward flavour
    for k in results["store_all"]:
        a, b = results["low_memory"][k], results["store_all"][k]
        assert _rel(a, b) < 1.6 * _rel(tf32[k], ref_grads[k]) + 2e-2, k


def test_low_memory_policy_keeps_less(cuda):
    from monet_b200 import runner
    torch.manual_seed(0)
    model = torchvision.models.resnet50(num_classes=10).to(cuda).train()
    x = torch.randn(8, 3, 96, 96, device=cuda)
    peaks = {}
    for policy in ("store_all", "low_memory"):
        r = runner.Runner(model, getattr(runner, policy))
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        out = r.forward(x)
        r.backward(torch.ones_like(out))
        torch.cuda.synchronize()
        peaks[policy] = torch.cuda.max_memory_allocated() - base
        for p in model.parameters():
            p.grad = None
    assert peaks["low_memory"] < peaks["store_all"], peaks


@pytest.mark.parametrize("policy", ["low_memory", "budget_10gb"])
def test_graphed_step_matches_eager(cuda, policy):
    """A training step captured as a CUDA graph and replayed on new batches follows the same
    trajectory as the executor called step by step (same kernels, same order).  Two runs of
    either kind already differ in the last bits (atomic accumulation order in the
    backward-filter splits, TF32 rounding of slightly different statistics), and training
    amplifies that, hence the convolution tolerance."""
    from monet_b200 import runner
    from monet_b200.lm_ops.softmax import SoftmaxCrossEntropy
    cl = torch.channels_last
    torch.manual_seed(11)
    base = torchvision.models.resnet18(num_classes=10).train()
    g = torch.Generator().manual_seed(5)
    batches = [(torch.randn(4, 3, 64, 64, generator=g), torch.randint(0, 10, (4,), generator=g))
               for _ in range(4)]

    def make():
        m = copy.deepcopy(base).to(cuda).to(memory_format=cl)
        opt = torch.optim.SGD(m.parameters(), lr=0.005, momentum=0.9)
        r = runner.Runner(m, getattr(runner, policy), fuse=True)
        return m, opt, r

    # eager trajectory; the graphed one spends its warm-up steps on the first batch too (the
    # capture itself records the step without running it)
    warm = 2
    m1, opt1, r1 = make()
    ce1 = SoftmaxCrossEntropy()
    eager_losses = []
    for i, (x, y) in enumerate([batches[0]] * warm + batches):
        for p in m1.parameters():
            p.grad = None
        out = r1.forward(x.to(cuda).contiguous(memory_format=cl))
        loss = ce1.forward(out, y.to(cuda))
        r1.backward(ce1.backward())
        opt1.step()
        if i >= warm:
            eager_losses.append(float(loss))

    m2, opt2, r2 = make()
    x0, y0 = batches[0]
    gs = runner.GraphedStep(r2, SoftmaxCrossEntropy(), opt2,
                            x0.to(cuda).contiguous(memory_format=cl), y0.to(cuda), warmup=warm)
    graph_losses = []
    for x, y in batches:
        loss = gs(x.to(cuda).contiguous(memory_format=cl), y.to(cuda))
        graph_losses.append(float(loss))
    torch.cuda.synchronize()
    assert all(l == l for l in graph_losses)
    for a, b in zip(graph_losses, eager_losses):
        assert abs(a - b) <= 4e-2 * max(1.0, abs(b)), (graph_losses, eager_losses)
    # the classifier and the first batch norm's running statistics after the same number of steps
    # (the convolution filters of a 4-image batch with random labels are too ill-conditioned to
    # compare between any two runs: batch norm makes their gradients differences of large terms)
    p1, p2 = dict(m1.named_parameters()), dict(m2.named_parameters())
    for k in ("fc.weight", "fc.bias"):
        assert _rel(p2[k].detach(), p1[k].detach()) < 5e-2, k
    b1, b2 = dict(m1.named_buffers()), dict(m2.named_buffers())
    for k in ("bn1.running_mean", "bn1.running_var"):
        assert _rel(b2[k], b1[k]) < 5e-2, k
    # the eager and the replayed run must agree on every buffer they touch, counters included
    assert int(b2["bn1.num_batches_tracked"]) == int(b1["bn1.num_batches_tracked"])
