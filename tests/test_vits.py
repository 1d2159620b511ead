"""VITS text-to-speech (``audio/vits.py``): parity with the Hugging Face implementation for synthesis, the monotonic
alignment against exhaustive search, and a training step that lowers its losses."""
import itertools

import pytest
import torch

from idrak_b200.audio import vits as V


def _tiny_hf(speakers=1):
    from transformers import VitsConfig, VitsModel
    cfg = VitsConfig(vocab_size=20, hidden_size=16, num_hidden_layers=2, num_attention_heads=2, window_size=2,
                     ffn_dim=32, flow_size=8, spectrogram_bins=9, duration_predictor_filter_channels=12,
                     prior_encoder_num_flows=2, prior_encoder_num_wavenet_layers=2, posterior_encoder_num_wavenet_layers=2,
                     wavenet_kernel_size=3, upsample_rates=[4, 2], upsample_kernel_sizes=[8, 4], upsample_initial_channel=16,
                     resblock_kernel_sizes=[3, 5], resblock_dilation_sizes=[[1, 3], [1, 2]],
                     use_stochastic_duration_prediction=False, noise_scale=0.0,
                     num_speakers=speakers, speaker_embedding_size=6 if speakers > 1 else 0)
    torch.manual_seed(0)
    model = VitsModel(cfg).eval()
    with torch.no_grad():                                   # durations of more than one frame, non-trivial weights
        model.duration_predictor.proj.bias.fill_(0.8)
        for p in model.parameters():
            if p.dim() > 1:
                p.mul_(1.5)
    return cfg, model


@pytest.mark.parametrize("speakers", [1, 3])
def test_synthesis_matches_the_hugging_face_model(speakers):
    cfg, hf = _tiny_hf(speakers)
    mine = V.Vits(V.VitsSpec.from_hf(cfg.to_dict())).eval()
    mine.load_hf_state(hf.state_dict())
    ids = torch.tensor([[3, 7, 1, 12, 5, 9, 2, 2, 15, 4, 11]])
    kw = {"speaker_id": 2} if speakers > 1 else {}
    with torch.no_grad():
        want = hf(ids, **kw)
    wave, samples = mine.synthesize(ids, speaker=torch.tensor([2]) if speakers > 1 else None, noise_scale=0.0)
    assert wave.shape == want.waveform.shape and int(samples[0]) == int(want.sequence_lengths[0])
    assert wave.shape[1] > 11 * 8                           # more than one frame per token somewhere
    torch.testing.assert_close(wave, want.waveform, atol=5e-4, rtol=1e-3)


def test_padded_batch_equals_single_sequences():
    cfg, hf = _tiny_hf()
    mine = V.Vits(V.VitsSpec.from_hf(cfg.to_dict())).eval()
    mine.load_hf_state(hf.state_dict())
    a, b = torch.tensor([[3, 7, 1, 12, 5, 9]]), torch.tensor([[4, 4, 8]])
    wa, na = mine.synthesize(a, noise_scale=0.0)
    wb, nb = mine.synthesize(b, noise_scale=0.0)
    batch = torch.tensor([[3, 7, 1, 12, 5, 9], [4, 4, 8, 0, 0, 0]])
    w, n = mine.synthesize(batch, lengths=torch.tensor([6, 3]), noise_scale=0.0)
    assert n.tolist() == [int(na), int(nb)]
    torch.testing.assert_close(w[0, :int(na)], wa[0], atol=1e-5, rtol=1e-4)
    # the shorter sequence: samples away from its end are untouched by the padding (the generator's receptive field)
    keep = int(nb) - 64
    torch.testing.assert_close(w[1, :keep], wb[0, :keep], atol=1e-5, rtol=1e-4)


def _best_by_enumeration(score):
    Fm, Tm = score.shape
    best, arg = None, None
    for cuts in itertools.combinations(range(1, Fm), Tm - 1):      # frame at which each next token starts
        bounds = (0,) + cuts + (Fm,)
        total = sum(score[f, t].item() for t in range(Tm) for f in range(bounds[t], bounds[t + 1]))
        if best is None or total > best:
            best, arg = total, bounds
    path = torch.zeros(Fm, Tm)
    for t in range(Tm):
        path[arg[t]:arg[t + 1], t] = 1
    return path, best


def test_monotonic_alignment_is_the_exhaustive_optimum():
    torch.manual_seed(1)
    score = torch.randn(3, 9, 4)
    frames, tokens = torch.tensor([9, 7, 4]), torch.tensor([4, 3, 4])
    path = V.monotonic_alignment(score, frames, tokens)
    for b in range(3):
        f, t = int(frames[b]), int(tokens[b])
        want, best = _best_by_enumeration(score[b, :f, :t])
        got = path[b, :f, :t]
        assert torch.equal(got.sum(1), torch.ones(f)) and bool((got.sum(0) >= 1).all())
        assert abs((got * score[b, :f, :t]).sum().item() - best) < 1e-5
        assert torch.equal(got, want)
        assert path[b, f:].sum() == 0 and path[b, :, t:].sum() == 0
    with pytest.raises(ValueError):
        V.monotonic_alignment(score, torch.tensor([2, 7, 4]), tokens)


def test_prior_scores_are_gaussian_log_densities():
    torch.manual_seed(2)
    z, mean, log_dev = torch.randn(2, 5, 7), torch.randn(2, 5, 3), 0.3 * torch.randn(2, 5, 3)
    got = V.prior_scores(z, mean, log_dev)
    dist = torch.distributions.Normal(mean[:, :, None, :], log_dev.exp()[:, :, None, :])
    want = dist.log_prob(z[:, :, :, None]).sum(1)
    torch.testing.assert_close(got, want, atol=1e-4, rtol=1e-4)


def test_flow_inverts_and_expansion_repeats_columns():
    spec = V.VitsSpec(vocab_size=10, hidden=16, layers=1, flow_size=8, spectrogram_bins=9, prior_flows=3,
                      prior_wavenet_layers=2, posterior_wavenet_layers=2, wavenet_kernel=3, upsample_rates=(2, 2),
                      upsample_kernels=(4, 4), upsample_channels=8, resblock_kernels=(3,), resblock_dilations=((1, 2),),
                      ffn=16, duration_filter=8, speakers=2, speaker_dim=4)
    torch.manual_seed(3)
    flow = V.Flow(spec)
    x, g = torch.randn(2, 8, 11), torch.randn(2, 4, 1)
    mask = V.length_mask(torch.tensor([11, 6]), 11)
    y = flow(x * mask, mask, g)
    torch.testing.assert_close(flow(y, mask, g, reverse=True), x * mask, atol=1e-5, rtol=1e-5)
    values = torch.arange(6.0).view(1, 2, 3)
    out, total = V.expand_by_durations(values, torch.tensor([[2, 0, 3]]))
    assert int(total) == 5 and out[0, 0].tolist() == [0, 0, 2, 2, 2] and out[0, 1].tolist() == [3, 3, 5, 5, 5]


def test_training_step_lowers_the_losses():
    spec = V.VitsSpec(vocab_size=12, hidden=16, layers=1, heads=2, window=2, ffn=32, flow_size=8, spectrogram_bins=17,
                      duration_filter=8, prior_flows=2, prior_wavenet_layers=2, posterior_wavenet_layers=2, wavenet_kernel=3,
                      upsample_rates=(4, 2), upsample_kernels=(8, 4), upsample_channels=16, resblock_kernels=(3,),
                      resblock_dilations=((1, 3),))
    torch.manual_seed(4)
    model = V.Vits(spec)
    disc = V.Discriminators(periods=(2, 3), period_channels=(4, 8), scale_width=4)
    hop = spec.hop
    t = torch.arange(40 * hop) / 400.0
    wave = torch.stack([torch.sin(2 * torch.pi * 30 * t), torch.sin(2 * torch.pi * 55 * t) * 0.5])
    lin = V.linear_spectrogram(wave, n_fft=32, hop=hop)
    assert lin.shape == (2, 17, 40)
    ids = torch.tensor([[1, 2, 3, 4, 5, 6], [7, 8, 9, 0, 0, 0]])
    id_len, spec_len = torch.tensor([6, 3]), torch.tensor([40, 31])
    opt_g = torch.optim.AdamW(model.parameters(), lr=2e-3)
    opt_d = torch.optim.AdamW(disc.parameters(), lr=2e-3)
    gen = torch.Generator().manual_seed(0)
    first = last = None
    for step in range(12):
        out = model.training_losses(ids, id_len, lin, spec_len, segment=8, generator=gen)
        frames = int(out["segment_frames"])
        assert out["segment_wave"].shape == (2, 1, frames * hop)
        assert torch.equal(out["alignment"].sum(2)[0], torch.ones(40)) and out["alignment"][1, 31:].sum() == 0
        real = V.slice_wave(wave, out["segment_start"], frames, hop)
        # discriminator step
        d_loss = V.discriminator_loss(disc(real), disc(out["segment_wave"].detach()))
        opt_d.zero_grad(); d_loss.backward(); opt_d.step()
        # generator step: spectral + KL + duration + adversarial + feature matching
        fake_scores, real_scores = disc(out["segment_wave"]), disc(real)
        spectral = (V.linear_spectrogram(out["segment_wave"][:, 0], 32, hop).log()
                    - V.linear_spectrogram(real[:, 0], 32, hop).log()).abs().mean()
        g_loss = (45 * spectral + out["kl"] + out["duration"] + V.generator_adversarial_loss(fake_scores)
                  + V.feature_matching_loss(real_scores, fake_scores))
        opt_g.zero_grad(); g_loss.backward(); opt_g.step()
        assert torch.isfinite(g_loss) and torch.isfinite(d_loss)
        value = (45 * spectral + out["kl"] + out["duration"]).item()
        first = value if first is None else first
        last = value
    assert last < first
    mel = V.mel_from_linear(lin, 16000, mels=10)
    assert mel.shape == (2, 10, 40) and torch.isfinite(mel).all()


@pytest.mark.parametrize("adversarial", [False, True])
def test_trainer_modes(adversarial):
    spec = V.VitsSpec(vocab_size=12, hidden=16, layers=1, heads=2, window=2, ffn=32, flow_size=8, spectrogram_bins=17,
                      duration_filter=8, prior_flows=2, prior_wavenet_layers=2, posterior_wavenet_layers=2, wavenet_kernel=3,
                      upsample_rates=(4, 2), upsample_kernels=(8, 4), upsample_channels=16, resblock_kernels=(3,),
                      resblock_dilations=((1, 3),))
    torch.manual_seed(5)
    model = V.Vits(spec)
    disc = V.Discriminators(periods=(2, 3), period_channels=(4, 8), scale_width=4) if adversarial else None
    trainer = V.VitsTrainer(model, disc, lr=2e-3, segment=8, mels=6 if adversarial else 0)
    t = torch.arange(40 * spec.hop) / 400.0
    wave = torch.stack([torch.sin(2 * torch.pi * 30 * t), torch.sin(2 * torch.pi * 55 * t) * 0.5])
    ids = torch.tensor([[1, 2, 3, 4, 5, 6], [7, 8, 9, 0, 0, 0]])
    reports = [trainer.step(ids, torch.tensor([6, 3]), wave, torch.tensor([40 * spec.hop, 30 * spec.hop])) for _ in range(10)]
    assert ("discriminator" in reports[0]) == adversarial and trainer.steps == 10
    key = lambda r: 45 * r["spectral"] + r["kl"] + r["duration"]
    assert key(reports[-1]) < key(reports[0])
    wave_out, samples = model.eval().synthesize(ids, torch.tensor([6, 3]))
    assert wave_out.shape[0] == 2 and int(samples.max()) == wave_out.shape[1]


def test_voice_conversion_is_the_identity_for_the_same_speaker_and_changes_with_the_target():
    spec = V.VitsSpec(vocab_size=10, hidden=16, layers=1, flow_size=8, spectrogram_bins=17, prior_flows=2,
                      prior_wavenet_layers=2, posterior_wavenet_layers=2, wavenet_kernel=3, upsample_rates=(2, 2),
                      upsample_kernels=(4, 4), upsample_channels=8, resblock_kernels=(3,), resblock_dilations=((1, 2),),
                      ffn=16, duration_filter=8, speakers=3, speaker_dim=4)
    torch.manual_seed(6)
    model = V.Vits(spec).eval()
    lin = torch.rand(2, 17, 12) + 0.1
    lengths = torch.tensor([12, 9])
    a, b = torch.tensor([0, 1]), torch.tensor([2, 2])
    same, n = model.convert_voice(lin, lengths, a, a)
    # same speaker in and out: the flow cancels, so it is posterior mean -> generator
    mask = V.length_mask(lengths, 12)
    g = model.embed_speaker(a).unsqueeze(-1)
    _, mean, _ = model.posterior_encoder(lin, mask, g)
    torch.testing.assert_close(same, model.decoder(mean * mask, g)[:, 0], atol=1e-5, rtol=1e-4)
    other, _ = model.convert_voice(lin, lengths, a, b)
    assert n.tolist() == [48, 36] and other.shape == same.shape and (other - same).abs().max() > 1e-4
    # a tone-colour embedding taken from a recording works in place of a speaker id
    ref = V.ReferenceEncoder(17, 4, channels=(4, 8), hidden=8)
    emb = ref(torch.rand(2, 17, 30))
    assert emb.shape == (2, 4, 1)
    cloned, _ = model.convert_voice(lin, lengths, a, emb)
    assert cloned.shape == same.shape and torch.isfinite(cloned).all()


def _tiny_hf_stochastic():
    from transformers import VitsConfig, VitsModel
    cfg = VitsConfig(vocab_size=20, hidden_size=16, num_hidden_layers=1, num_attention_heads=2, window_size=2,
                     ffn_dim=32, flow_size=8, spectrogram_bins=9, prior_encoder_num_flows=2,
                     prior_encoder_num_wavenet_layers=2, posterior_encoder_num_wavenet_layers=2, wavenet_kernel_size=3,
                     upsample_rates=[4, 2], upsample_kernel_sizes=[8, 4], upsample_initial_channel=16,
                     resblock_kernel_sizes=[3], resblock_dilation_sizes=[[1, 3]], use_stochastic_duration_prediction=True,
                     duration_predictor_num_flows=3, duration_predictor_flow_bins=5, depth_separable_num_layers=2,
                     noise_scale=0.0, noise_scale_duration=0.0)
    torch.manual_seed(0)
    model = VitsModel(cfg).eval()
    with torch.no_grad():
        for name, p in model.duration_predictor.named_parameters():
            if p.dim() > 1 and "norm" not in name:
                p.mul_(3.0)
        model.duration_predictor.flows[0].translate.add_(torch.tensor([[0.9], [0.2]]))
        model.duration_predictor.flows[0].log_scale.add_(torch.tensor([[0.3], [-0.2]]))
    return cfg, model


def test_stochastic_duration_predictor_matches_hugging_face():
    cfg, hf = _tiny_hf_stochastic()
    mine = V.Vits(V.VitsSpec.from_hf(cfg.to_dict())).eval()
    mine.load_hf_state(hf.state_dict())
    ids = torch.tensor([[3, 7, 1, 12, 5, 9, 2, 15]])
    with torch.no_grad():
        want = hf(ids)
    wave, samples = mine.synthesize(ids, noise_scale=0.0, noise_scale_duration=0.0)
    assert wave.shape == want.waveform.shape and wave.shape[1] > 8 * 8
    torch.testing.assert_close(wave, want.waveform, atol=5e-4, rtol=1e-3)
    # the training bound, same noise
    x, mask = torch.randn(2, 16, 6), V.length_mask(torch.tensor([6, 4]), 6)
    durations = torch.tensor([[[2., 1, 3, 1, 4, 2]], [[1., 5, 2, 2, 0, 0]]]) * mask
    torch.manual_seed(11)
    with torch.no_grad():
        want_nll = hf.duration_predictor(x, mask, None, durations=durations, reverse=False)
    torch.manual_seed(11)
    with torch.no_grad():
        got_nll = mine.duration_predictor.negative_log_likelihood(x, mask, durations)
    torch.testing.assert_close(got_nll, want_nll, atol=1e-3, rtol=1e-4)


def test_spline_is_monotone_invertible_and_reports_its_slope():
    torch.manual_seed(12)
    x = (torch.randn(3, 1, 40, dtype=torch.double) * 3).requires_grad_(True)
    w, h, d = (torch.randn(3, 1, 40, n, dtype=torch.double) for n in (6, 6, 5))
    y, logdet = V.rational_quadratic_spline(x, w, h, d)
    slope, = torch.autograd.grad(y.sum(), x)
    torch.testing.assert_close(slope.log(), logdet, atol=1e-9, rtol=1e-9)
    back, _ = V.rational_quadratic_spline(y.detach(), w, h, d, inverse=True)
    torch.testing.assert_close(back, x.detach(), atol=1e-9, rtol=1e-9)
    outside = x.detach().abs() > 5
    assert bool(outside.any()) and torch.equal(y.detach()[outside], x.detach()[outside])


def test_training_with_the_stochastic_duration_model():
    spec = V.VitsSpec(vocab_size=12, hidden=16, layers=1, heads=2, window=2, ffn=32, flow_size=8, spectrogram_bins=17,
                      prior_flows=2, prior_wavenet_layers=2, posterior_wavenet_layers=2, wavenet_kernel=3,
                      upsample_rates=(4, 2), upsample_kernels=(8, 4), upsample_channels=16, resblock_kernels=(3,),
                      resblock_dilations=((1, 3),), stochastic_duration=True, duration_flows=2, duration_flow_bins=4,
                      duration_stack_layers=2, duration_dropout=0.0)
    torch.manual_seed(13)
    model = V.Vits(spec)
    trainer = V.VitsTrainer(model, None, lr=2e-3, segment=8)
    t = torch.arange(40 * spec.hop) / 400.0
    wave = torch.stack([torch.sin(2 * torch.pi * 30 * t), torch.sin(2 * torch.pi * 55 * t) * 0.5])
    ids = torch.tensor([[1, 2, 3, 4, 5, 6], [7, 8, 9, 0, 0, 0]])
    reports = [trainer.step(ids, torch.tensor([6, 3]), wave, torch.tensor([40 * spec.hop, 30 * spec.hop])) for _ in range(15)]
    assert all(torch.isfinite(torch.tensor(r["loss"])) for r in reports)
    assert sum(r["duration"] for r in reports[-3:]) < sum(r["duration"] for r in reports[:3])
    wave_out, samples = model.eval().synthesize(ids, torch.tensor([6, 3]))
    assert int(samples.max()) == wave_out.shape[1]
