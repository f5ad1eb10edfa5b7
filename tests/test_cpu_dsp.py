"""Signal-processing routines against scipy / numpy statements of the same definitions (CPU)."""
import math

import numpy as np
import pytest
import torch

from scirust_b200 import dsp as D

ss = pytest.importorskip("scipy.signal")


@pytest.fixture(scope="module")
def x():
    return torch.randn(3, 2048, dtype=torch.float64, generator=torch.Generator().manual_seed(0))


def test_periodic_windows_match_scipy():
    for name, fn in (("hann", D.hann), ("hamming", D.hamming), ("blackman", D.blackman)):
        assert np.abs(fn(64, torch.float64).numpy() - ss.get_window(name, 64, fftbins=True)).max() < 1e-12
    assert float(D.kaiser(32, 0.0, torch.float64).min()) == 1.0                       # beta 0 is the rectangular window
    bh = D.blackman_harris(128, torch.float64)
    assert abs(float(bh[0]) - 0.0) < 1e-12 and abs(float(bh[64]) - 1.0) < 1e-12
    with pytest.raises(ValueError):
        D.hann(0)


def test_stft_round_trip_welch_and_convolution(x):
    w = D.hann(256, torch.float64)
    z = D.stft(x, w, 128)
    assert z.shape == (3, D.num_frames(2048, 256, 128), 129)
    y = D.istft(z, 256, 128)
    assert float((y[..., 256:-256] - x[..., 256:y.shape[-1] - 256]).abs().max()) < 1e-12       # Hann at 50 % is COLA
    _, p = ss.welch(x[0].numpy(), fs=1000.0, window=w.numpy(), nperseg=256, noverlap=128, detrend=False)
    assert np.abs(D.welch(x, w, 128, 1000.0)[0].numpy() - p).max() < 1e-12 * p.max() + 1e-15
    assert float(D.welch_freqs(256, 1000.0)[-1]) == 500.0
    k = torch.randn(31, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    ref = np.convolve(x[0].numpy(), k.numpy())
    assert np.abs(D.fft_convolve(x, k)[0].numpy() - ref).max() < 1e-10
    assert np.abs(D.fft_convolve(x, k, 128)[0].numpy() - ref).max() < 1e-10                     # overlap-add blocks
    with pytest.raises(ValueError):
        D.num_frames(100, 256, 128)
    with pytest.raises(ValueError):
        D.fft_convolve(x, k, 16)


def test_goertzel_is_the_dft_at_any_frequency_and_hilbert_matches_scipy(x):
    spec = np.fft.fft(x[1].numpy())
    g = D.goertzel(x, torch.tensor([2 * math.pi * 5 / 2048, 2 * math.pi * 100 / 2048], dtype=torch.float64))
    assert abs(complex(g[1, 0]) - spec[5]) < 1e-9 and abs(complex(g[1, 1]) - spec[100]) < 1e-9
    assert abs(float(D.goertzel_power(x, 2 * math.pi * 5 / 2048)[1]) - abs(spec[5]) ** 2) < 1e-7
    assert np.abs(D.analytic_signal(x)[0].numpy() - ss.hilbert(x[0].numpy())).max() < 1e-12
    n = torch.arange(4096, dtype=torch.float64)
    tone = torch.cos(2 * math.pi * 50.0 * n / 1000.0)
    f = D.instantaneous_frequency(tone, 1000.0)
    assert float((f[200:-200] - 50.0).abs().max()) < 0.5 and float((D.envelope(tone)[200:-200] - 1).abs().max()) < 0.02


def test_biquad_cascades_match_scipy_designs_and_stream_without_seams(x):
    cases = [(D.BiquadCascade.butterworth_lowpass(1000.0, 100.0, 4), ss.butter(4, 100.0, fs=1000.0, output="sos")),
             (D.BiquadCascade.butterworth_highpass(1000.0, 100.0, 6), ss.butter(6, 100.0, "high", fs=1000.0, output="sos")),
             (D.BiquadCascade.chebyshev1_lowpass(1000.0, 100.0, 4, 1.0), ss.cheby1(4, 1.0, 100.0, fs=1000.0, output="sos")),
             (D.BiquadCascade.chebyshev1_highpass(1000.0, 100.0, 4, 1.0), ss.cheby1(4, 1.0, 100.0, "high", fs=1000.0, output="sos"))]
    for cascade, sos in cases:
        y = cascade.process_block(x)
        for r in range(3):
            assert np.abs(y[r].numpy() - ss.sosfilt(sos, x[r].numpy())).max() < 1e-10
    c = D.BiquadCascade.butterworth_lowpass(1000.0, 100.0, 4)
    whole = c.process_block(x)
    c.reset()
    parts = torch.cat([c.process_block(x[:, :1000]), c.process_block(x[:, 1000:])], -1)
    assert torch.equal(whole, parts)
    h = c.frequency_response(torch.tensor(2 * math.pi * 100.0 / 1000.0))
    assert abs(float(D.magnitude_db(h)) + 3.0103) < 1e-3 and c.order() == 4                     # -3 dB at the corner
    with pytest.raises(ValueError):
        D.butterworth_qs(3)
    bp = D.Biquad.bandpass(1000.0, 100.0, 5.0)
    assert abs(abs(complex(bp.frequency_response(2 * math.pi * 0.1))) - 5.0) < 1e-9          # constant-skirt form: peak gain = Q


def test_fir_savgol_dct_wavelets_and_resampling(x):
    k = torch.randn(31, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    fir = D.Fir(k)
    y = torch.cat([fir.process_block(x[:, :700]), fir.process_block(x[:, 700:])], -1)
    assert np.abs(y[0].numpy() - ss.lfilter(k.numpy(), [1.0], x[0].numpy())).max() < 1e-10
    assert np.abs(D.savgol_filter(x, 11, 3)[0].numpy() - ss.savgol_filter(x[0].numpy(), 11, 3, mode="nearest")).max() < 1e-10
    assert np.abs(D.savgol_coeffs(7, 2, 1).numpy() - ss.savgol_coeffs(7, 2, deriv=1, use="dot")).max() < 1e-12
    from scipy.fft import dct
    assert np.abs(D.dct2(x[:, :40]).numpy() - dct(x[:, :40].numpy(), type=2, norm="ortho")).max() < 1e-12
    for wv in ("haar", "cdf53"):
        coeffs = D.dwt_decompose(x, 3, wv)
        assert float((D.dwt_reconstruct(coeffs, 3, wv) - x).abs().max()) < 1e-12
    ramp = torch.arange(64, dtype=torch.float64)
    assert float(D.dwt_decompose(ramp, 1, "cdf53")[32:-1].abs().max()) < 1e-12                    # linear signals have no detail
    with pytest.raises(ValueError):
        D.dwt_decompose(x[:, :100], 3)
    n = torch.arange(1000, dtype=torch.float64)
    r = D.resample(torch.sin(2 * math.pi * 0.01 * n), 3, 2, 8)
    m = torch.arange(r.shape[-1], dtype=torch.float64)
    assert r.shape[-1] == 1500 and float((r - torch.sin(2 * math.pi * 0.01 * m * 2 / 3))[50:-50].abs().max()) < 1e-3


def test_mel_filterbank_mfcc_and_log_mel_features(x):
    fb = D.MelFilterbank(26, 129, 16000.0, 0.0, 8000.0, torch.float64)
    assert fb.weights.shape == (26, 129) and float(fb.weights.min()) >= 0.0 and float(fb.weights.max()) <= 1.0
    assert bool((fb.weights.sum(1) > 0).all())
    peaks = fb.weights.argmax(1)
    assert bool((peaks[1:] >= peaks[:-1]).all())                                                  # centres rise with the band
    p = D.power_spectrogram(D.stft(x, D.hann(256, torch.float64), 128))
    mf = D.Mfcc(26, 13, 129, 16000.0, 0.0, 8000.0, torch.float64)
    out = mf.apply(p)
    assert out.shape == (3, 15, 13) and bool(torch.isfinite(out).all())
    assert torch.allclose(out, (torch.log(fb.apply(p)) @ D.dct2_basis(13, 26, torch.float64).t()))
    assert D.log_mel_features(x.float(), 16000.0).shape == (3, 7, 40)
    with pytest.raises(ValueError):
        D.Mfcc(13, 26, 129, 16000.0, 0.0, 8000.0)


def test_adaptive_filters_identify_a_system_kalman_tracks_and_pll_locks():
    g = torch.Generator().manual_seed(3)
    xs = torch.randn(1500, dtype=torch.float64, generator=g)
    h = torch.tensor([0.5, -0.3, 0.2, 0.1], dtype=torch.float64)
    d = torch.from_numpy(np.convolve(xs.numpy(), h.numpy())[:1500])
    for filt, tol in ((D.Lms(4, 0.02), 2e-2), (D.Nlms(4, 0.5), 1e-3), (D.Rls(4, 0.999, 100.0), 1e-5)):
        _, err = filt.run(xs, d)
        assert float((filt.weights - h).abs().max()) < tol and float(err[-50:].abs().max()) < 10 * tol
    kf = D.KalmanFilter([0.0, 0.0], torch.eye(2) * 10.0)
    f, q = torch.tensor([[1.0, 1.0], [0.0, 1.0]]), torch.eye(2) * 1e-6
    hm, r = torch.tensor([[1.0, 0.0]]), torch.tensor([[0.04]])
    noise = 0.2 * torch.randn(200, dtype=torch.float64, generator=g)
    for t in range(200):
        kf.predict(f, q)
        assert kf.update(torch.tensor([3.0 + 0.5 * (t + 1)]) + noise[t], hm, r)
    assert abs(float(kf.x[1]) - 0.5) < 0.01 and abs(float(kf.x[0]) - (3.0 + 0.5 * 200)) < 0.3
    pll = D.Pll(8000.0, 1000.0, 100.0)
    for t in range(4000):
        ph = 2 * math.pi * 1010.0 * t / 8000.0
        pll.process_quadrature(math.cos(ph), math.sin(ph))
    assert abs(pll.frequency_estimate() - 1010.0) < 0.5 and pll.locked(1e-3)
