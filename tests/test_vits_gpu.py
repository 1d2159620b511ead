"""VITS on the device: the bf16 model (1-D convolutions on this package's kernels) against the fp32 CPU model."""
import pytest
import torch

from idrak_b200.audio import vits as V

pytestmark = pytest.mark.gpu


def _spec():
    return V.VitsSpec(vocab_size=24, hidden=64, layers=2, heads=2, window=4, ffn=128, flow_size=32, spectrogram_bins=65,
                      duration_filter=64, prior_flows=2, prior_wavenet_layers=2, posterior_wavenet_layers=3, wavenet_kernel=5,
                      upsample_rates=(4, 4), upsample_kernels=(8, 8), upsample_channels=64, resblock_kernels=(3, 7),
                      resblock_dilations=((1, 3), (1, 3)))


def _rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).norm() / b.float().cpu().norm()).item()


def test_generator_flow_and_posterior_in_bf16_follow_the_fp32_cpu_model():
    torch.manual_seed(0)
    cpu = V.Vits(_spec()).eval()
    dev = V.Vits(_spec()).eval()
    dev.load_state_dict(cpu.state_dict())
    dev = dev.cuda().bfloat16()
    z = torch.randn(2, 32, 48)
    mask = V.length_mask(torch.tensor([48, 30]), 48)
    with torch.no_grad():
        assert _rel(dev.decoder(z.cuda().bfloat16()), cpu.decoder(z)) < 0.05
        want = cpu.flow(z * mask, mask)
        got = dev.flow((z * mask).cuda().bfloat16(), mask.cuda().bfloat16())
        assert _rel(got, want) < 0.03
        back = dev.flow(got, mask.cuda().bfloat16(), reverse=True)
        assert _rel(back, z * mask) < 0.03
        lin = torch.rand(2, 65, 48) + 0.1
        _, mean_c, dev_c = cpu.posterior_encoder(lin, mask)
        _, mean_d, dev_d = dev.posterior_encoder(lin.cuda().bfloat16(), mask.cuda().bfloat16())
        assert _rel(mean_d, mean_c) < 0.05 and _rel(dev_d, dev_c) < 0.05
        ids = torch.randint(1, 24, (2, 12))
        tmask = V.length_mask(torch.tensor([12, 9]), 12)
        h_c, m_c, _ = cpu.text_encoder(ids, tmask)
        h_d, m_d, _ = dev.text_encoder(ids.cuda(), tmask.cuda().bfloat16())
        assert _rel(h_d, h_c) < 0.05 and _rel(m_d, m_c) < 0.06
        wave, samples = dev.synthesize(ids.cuda(), torch.tensor([12, 9], device="cuda"))
        assert wave.dtype == torch.bfloat16 and int(samples.max()) == wave.shape[1] and torch.isfinite(wave.float()).all()


def test_training_step_and_synthesis_run_on_the_device():
    torch.manual_seed(1)
    spec = _spec()
    model = V.Vits(spec).cuda()
    trainer = V.VitsTrainer(model, V.Discriminators(periods=(2, 3), period_channels=(8, 16), scale_width=4).cuda(),
                            lr=1e-3, segment=8)
    trainer.generator = torch.Generator(device="cuda").manual_seed(0)
    t = torch.arange(40 * spec.hop, device="cuda") / 800.0
    wave = torch.stack([torch.sin(2 * torch.pi * 60 * t), 0.5 * torch.sin(2 * torch.pi * 95 * t)])
    ids = torch.tensor([[1, 2, 3, 4, 5, 6], [7, 8, 9, 0, 0, 0]], device="cuda")
    lengths = torch.tensor([6, 3], device="cuda")
    reports = [trainer.step(ids, lengths, wave, torch.tensor([40 * spec.hop, 30 * spec.hop], device="cuda"))
               for _ in range(6)]
    assert all(r["loss"] == r["loss"] for r in reports)
    key = lambda r: 45 * r["spectral"] + r["kl"] + r["duration"]
    assert key(reports[-1]) < key(reports[0])
    out, samples = model.eval().synthesize(ids, lengths, generator=torch.Generator(device="cuda").manual_seed(2))
    assert out.is_cuda and int(samples.max()) == out.shape[1] and torch.isfinite(out).all()


def test_alignment_kernel_equals_the_host_search():
    torch.manual_seed(3)
    score = torch.randn(5, 70, 23)
    frames, tokens = torch.tensor([70, 51, 23, 64, 30]), torch.tensor([23, 17, 23, 1, 9])
    want = V.monotonic_alignment(score, frames, tokens)
    got = V.monotonic_alignment(score.cuda(), frames.cuda(), tokens.cuda())
    assert got.is_cuda and torch.equal(got.cpu(), want)
    # scores with many ties (the same choice on both sides)
    tied = torch.randint(0, 3, (2, 40, 11)).float()
    f2, t2 = torch.tensor([40, 33]), torch.tensor([11, 8])
    assert torch.equal(V.monotonic_alignment(tied.cuda(), f2.cuda(), t2.cuda()).cpu(), V.monotonic_alignment(tied, f2, t2))
