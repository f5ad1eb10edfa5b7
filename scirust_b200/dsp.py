"""Signal processing on torch tensors: every routine works on the LAST axis and is batched over the leading ones, on
whichever device the input lives (FFTs go to cuFFT on a GPU), so a whole batch of audio clips becomes log-mel or MFCC
features without a host round trip.

Windows are PERIODIC (angle 2*pi*n/len: the analysis form, COLA at 50 % overlap for Hann). ``stft`` frames without
padding (``num_frames = (len - frame) // hop + 1``) and returns ``[..., frames, frame/2 + 1]``; ``istft`` is a plain
overlap-add of the inverse transforms (exact up to the edges when the analysis window is COLA at that hop). The mel
scale is the HTK one (2595 log10(1 + f/700)), triangles are unnormalised; the DCT-II is orthonormal; MFCC = DCT of the
natural log of the mel energies with no floor. ``welch`` is the one-sided density 1/(fs * sum w^2), interior bins doubled.
``goertzel`` returns sum x[n] exp(-j omega n) (the DFT at an arbitrary frequency) as a batched matrix product. Biquads
are RBJ designs run as a cascade (Butterworth / Chebyshev-I sections of even order, bilinear via per-section Q);
recursive filters run in a native loop on CPU tensors and as a time loop vectorised over the batch elsewhere.
Wavelets use lifting (Haar, CDF 5/3 with symmetric edge handling), in place-order [approximation | detail].
Reference counterpart: scirust-simd/src/dsp/{window,fft,fftconv,stft,mel,mfcc,welch,goertzel,hilbert,fir,biquad,freqz,
savgol,resample,wavelet,adaptive,kalman,pll}.rs.
"""
from __future__ import annotations

import math

import torch


def _t(x, dtype=None):
    x = torch.as_tensor(x)
    if not (x.is_floating_point() or x.is_complex()):
        x = x.to(torch.float32)
    return x.to(dtype) if dtype is not None else x


# ------------------------------------------------------------------ windows (periodic)
def _angle(n_len, dtype, device):
    if n_len < 1:
        raise ValueError("a window needs at least one sample")
    return 2.0 * math.pi * torch.arange(n_len, dtype=dtype, device=device) / n_len


def hann(n, dtype=torch.float32, device=None):
    return 0.5 - 0.5 * torch.cos(_angle(n, dtype, device))


def hamming(n, dtype=torch.float32, device=None):
    return 0.54 - 0.46 * torch.cos(_angle(n, dtype, device))


def blackman(n, dtype=torch.float32, device=None):
    th = _angle(n, dtype, device)
    return 0.42 - 0.5 * torch.cos(th) + 0.08 * torch.cos(2 * th)


def blackman_harris(n, dtype=torch.float32, device=None):
    th = _angle(n, dtype, device)
    return 0.36 - 0.49 * torch.cos(th) + 0.14 * torch.cos(2 * th) - 0.01 * torch.cos(3 * th)


def kaiser(n, beta, dtype=torch.float32, device=None):
    if n < 1:
        raise ValueError("a window needs at least one sample")
    r = torch.arange(n, dtype=torch.float64, device=device) * (2.0 / n) - 1.0
    b = torch.tensor(float(beta), dtype=torch.float64, device=device)
    return (torch.special.i0(b * torch.sqrt((1.0 - r * r).clamp_min(0.0))) / torch.special.i0(b)).to(dtype)


# ------------------------------------------------------------------ transforms
def fft(x):
    return torch.fft.fft(_t(x))


def ifft(x):
    return torch.fft.ifft(_t(x))


def rfft(x):
    return torch.fft.rfft(_t(x))


def irfft(x, n):
    return torch.fft.irfft(_t(x), n=n)


def fft_convolve(signal, kernel, fft_size: int | None = None):
    """Full linear convolution (length ``n + k - 1``). With ``fft_size`` the signal is processed in overlap-add blocks of
    ``fft_size - k + 1`` samples (constant memory per block, all blocks transformed as one batch)."""
    s, k = _t(signal), _t(kernel)
    n, m = s.shape[-1], k.shape[-1]
    if n == 0 or m == 0:
        raise ValueError("empty operand")
    full = n + m - 1
    if fft_size is None:
        size = 1 << (full - 1).bit_length()
        return torch.fft.irfft(torch.fft.rfft(s, n=size) * torch.fft.rfft(k, n=size), n=size)[..., :full]
    if fft_size < m or fft_size & (fft_size - 1):
        raise ValueError("fft_size must be a power of two and at least the kernel length")
    step = fft_size - m + 1
    blocks = -(-n // step)
    pad = torch.nn.functional.pad(s, (0, blocks * step - n)).reshape(*s.shape[:-1], blocks, step)
    seg = torch.fft.irfft(torch.fft.rfft(pad, n=fft_size) * torch.fft.rfft(k, n=fft_size)[..., None, :], n=fft_size)
    out = s.new_zeros(*s.shape[:-1], blocks * step + m - 1)
    idx = (torch.arange(blocks, device=s.device)[:, None] * step + torch.arange(fft_size, device=s.device)[None, :]).reshape(-1)
    out.index_add_(-1, idx, seg.reshape(*s.shape[:-1], -1))
    return out[..., :full]


def num_frames(signal_len: int, frame_size: int, hop: int) -> int:
    if hop < 1:
        raise ValueError("hop must be at least 1")
    if signal_len < frame_size:
        raise ValueError(f"signal of length {signal_len} is shorter than one frame of {frame_size}")
    return (signal_len - frame_size) // hop + 1


def stft(signal, window, hop: int):
    x, w = _t(signal), _t(window)
    frames = num_frames(x.shape[-1], w.shape[-1], hop)
    return torch.fft.rfft(x.unfold(-1, w.shape[-1], hop)[..., :frames, :] * w.to(x.device))


def istft(spectrogram, frame_size: int, hop: int):
    z = _t(spectrogram)
    if z.shape[-1] != frame_size // 2 + 1:
        raise ValueError(f"expected {frame_size // 2 + 1} bins per frame")
    t = torch.fft.irfft(z, n=frame_size)
    frames = t.shape[-2]
    out = t.new_zeros(*t.shape[:-2], (frames - 1) * hop + frame_size)
    idx = (torch.arange(frames, device=t.device)[:, None] * hop + torch.arange(frame_size, device=t.device)[None, :]).reshape(-1)
    return out.index_add_(-1, idx, t.reshape(*t.shape[:-2], -1))


def power_spectrogram(z):
    return z.real ** 2 + z.imag ** 2


def magnitude_spectrogram(z):
    return z.abs()


# ------------------------------------------------------------------ mel / MFCC
def hz_to_mel(hz):
    return 2595.0 * math.log10(1.0 + hz / 700.0)


def mel_to_hz(mel):
    return 700.0 * (10.0 ** (mel / 2595.0) - 1.0)


class MelFilterbank:
    def __init__(self, n_mels: int, bins: int, sample_rate: float, f_min: float, f_max: float, dtype=torch.float32):
        if n_mels < 1 or bins < 2 or not f_min < f_max:
            raise ValueError("need n_mels >= 1, bins >= 2 and f_min < f_max")
        lo, hi = hz_to_mel(f_min), hz_to_mel(f_max)
        pts = torch.tensor([mel_to_hz(lo + i * (hi - lo) / (n_mels + 1)) for i in range(n_mels + 2)], dtype=torch.float64)
        f = torch.arange(bins, dtype=torch.float64) * (sample_rate / (2 * (bins - 1)))
        left, centre, right = pts[:-2, None], pts[1:-1, None], pts[2:, None]
        up, down = (f - left) / (centre - left), (right - f) / (right - centre)
        w = torch.where(f <= centre, up, down)
        self.weights = torch.where((f <= left) | (f >= right), torch.zeros_like(w), w).to(dtype)      # [n_mels, bins]
        self.n_mels, self.bins = n_mels, bins

    def apply(self, spectrogram):
        s = _t(spectrogram)
        if s.shape[-1] != self.bins:
            raise ValueError(f"expected {self.bins} bins per frame, got {s.shape[-1]}")
        return s @ self.weights.to(s.device, s.dtype).t()


def dct2_basis(n_coeffs: int, n: int, dtype=torch.float32):
    k = torch.arange(n_coeffs, dtype=torch.float64)[:, None]
    m = torch.arange(n, dtype=torch.float64)[None, :]
    alpha = torch.where(k == 0, torch.tensor(math.sqrt(1.0 / n), dtype=torch.float64), torch.tensor(math.sqrt(2.0 / n), dtype=torch.float64))
    return (alpha * torch.cos(math.pi / n * (m + 0.5) * k)).to(dtype)


def dct2(x):
    x = _t(x)
    return x @ dct2_basis(x.shape[-1], x.shape[-1], x.dtype).to(x.device).t()


class Mfcc:
    def __init__(self, n_mels, n_coeffs, bins, sample_rate, f_min, f_max, dtype=torch.float32):
        if not 1 <= n_coeffs <= n_mels:
            raise ValueError("need 1 <= n_coeffs <= n_mels")
        self.filterbank = MelFilterbank(n_mels, bins, sample_rate, f_min, f_max, dtype)
        self.basis = dct2_basis(n_coeffs, n_mels, dtype)
        self.n_coeffs = n_coeffs

    def apply(self, spectrogram):
        mel = self.filterbank.apply(spectrogram)
        return torch.log(mel) @ self.basis.to(mel.device, mel.dtype).t()


def log_mel_features(signal, sample_rate: float, frame: int = 512, hop: int = 256, n_mels: int = 40, floor: float = 1e-10):
    """Waveforms ``[..., samples]`` -> ``[..., frames, n_mels]`` log-mel energies (Hann analysis window)."""
    x = _t(signal)
    p = power_spectrogram(stft(x, hann(frame, x.dtype, x.device), hop))
    return torch.log(MelFilterbank(n_mels, frame // 2 + 1, sample_rate, 0.0, sample_rate / 2, x.dtype).apply(p).clamp_min(floor))


# ------------------------------------------------------------------ spectral estimation
def welch(signal, window, hop: int, sample_rate: float):
    x, w = _t(signal), _t(window)
    p = power_spectrogram(stft(x, w, hop)).mean(-2) / (sample_rate * float((w.double() ** 2).sum()))
    scale = torch.full((p.shape[-1],), 2.0, dtype=p.dtype, device=p.device)
    scale[0] = 1.0
    if w.shape[-1] % 2 == 0:
        scale[-1] = 1.0
    return p * scale


def welch_freqs(frame: int, sample_rate: float):
    return torch.arange(frame // 2 + 1, dtype=torch.float64) * (sample_rate / frame)


def goertzel(x, omega):
    """``sum_n x[n] exp(-j omega n)`` for one or many ``omega`` (radians per sample) -> ``[..., len(omega)]`` complex."""
    x = _t(x)
    om = torch.as_tensor(omega, dtype=torch.float64, device=x.device).reshape(-1)
    n = torch.arange(x.shape[-1], dtype=torch.float64, device=x.device)
    ph = om[:, None] * n[None, :]
    ct = torch.complex64 if x.dtype == torch.float32 else torch.complex128
    out = x.to(ct) @ torch.complex(ph.cos(), -ph.sin()).to(ct).t()
    return out[..., 0] if torch.as_tensor(omega).dim() == 0 else out


def goertzel_power(x, omega):
    z = goertzel(x, omega)
    return z.real ** 2 + z.imag ** 2


def goertzel_hz(x, sample_rate, freq_hz):
    return goertzel(x, 2.0 * math.pi * torch.as_tensor(freq_hz, dtype=torch.float64) / sample_rate)


def analytic_signal(x):
    x = _t(x)
    n = x.shape[-1]
    h = torch.zeros(n, dtype=x.dtype, device=x.device)
    h[0] = 1.0
    if n % 2 == 0:
        h[n // 2] = 1.0
        h[1:n // 2] = 2.0
    else:
        h[1:(n + 1) // 2] = 2.0
    return torch.fft.ifft(torch.fft.fft(x) * h)


def hilbert(x):
    return analytic_signal(x).imag


def envelope(x):
    return analytic_signal(x).abs()


def instantaneous_phase(x):
    return torch.angle(analytic_signal(x))


def unwrap_phase(ph):
    ph = _t(ph)
    d = ph[..., 1:] - ph[..., :-1]
    wrapped = torch.remainder(d + math.pi, 2 * math.pi) - math.pi
    wrapped = torch.where((wrapped == -math.pi) & (d > 0), torch.full_like(wrapped, math.pi), wrapped)
    return torch.cat([ph[..., :1], ph[..., :1] + torch.cumsum(wrapped, -1)], -1)


def instantaneous_frequency(x, sample_rate: float):
    ph = unwrap_phase(instantaneous_phase(x))
    return (ph[..., 1:] - ph[..., :-1]) * (sample_rate / (2 * math.pi))


# ------------------------------------------------------------------ FIR / IIR
class Fir:
    """Streaming FIR: ``process_block`` keeps the last ``taps - 1`` inputs, so blocks concatenate seamlessly."""

    def __init__(self, taps):
        self.taps = _t(taps).reshape(-1)
        self.reset()

    def reset(self):
        self.state = None

    def process_block(self, x):
        x = _t(x, self.taps.dtype)
        k = self.taps.shape[0]
        hist = self.state if self.state is not None else x.new_zeros(*x.shape[:-1], k - 1)
        ext = torch.cat([hist, x], -1)
        self.state = ext[..., ext.shape[-1] - (k - 1):]
        return (ext.unfold(-1, k, 1) * self.taps.to(x.device).flip(0)).sum(-1)

    def frequency_response(self, omega):
        om = torch.as_tensor(omega, dtype=torch.float64).reshape(-1)
        k = torch.arange(self.taps.shape[0], dtype=torch.float64)
        return (torch.polar(torch.ones_like(om)[:, None].expand(-1, k.shape[0]), -om[:, None] * k) * self.taps.double()).sum(-1)


def _sos_filter(sos, x, state=None):
    """Direct form I cascade over the last axis. ``sos [sections, 5]`` = (b0, b1, b2, a1, a2); ``state [..., sections, 4]``
    = (x1, x2, y1, y2). Returns (y, state)."""
    x64 = x.to(torch.float64)
    lead = x64.shape[:-1]
    st = x64.new_zeros(*lead, sos.shape[0], 4) if state is None else state.to(torch.float64).clone()
    if x64.device.type == "cpu":
        from .cpu_kernels import sos_filter_native
        y = sos_filter_native(sos.double().contiguous(), x64.contiguous().reshape(-1, x64.shape[-1]), st.reshape(-1, sos.shape[0], 4))
        return y.reshape(x64.shape).to(x.dtype), st
    cur = x64
    for s in range(sos.shape[0]):
        b0, b1, b2, a1, a2 = (float(v) for v in sos[s])
        x1, x2, y1, y2 = st[..., s, 0].clone(), st[..., s, 1].clone(), st[..., s, 2].clone(), st[..., s, 3].clone()
        out = torch.empty_like(cur)
        for t in range(cur.shape[-1]):
            xt = cur[..., t]
            yt = b0 * xt + b1 * x1 + b2 * x2 - a1 * y1 - a2 * y2
            x2, x1, y2, y1 = x1, xt, y1, yt
            out[..., t] = yt
        st[..., s, 0], st[..., s, 1], st[..., s, 2], st[..., s, 3] = x1, x2, y1, y2
        cur = out
    return cur.to(x.dtype), st


class Biquad:
    def __init__(self, b0, b1, b2, a1, a2):
        self.coefficients = (float(b0), float(b1), float(b2), float(a1), float(a2))
        self.state = None

    @staticmethod
    def identity():
        return Biquad(1, 0, 0, 0, 0)

    @staticmethod
    def _prelude(fs, fc, q):
        w0 = 2.0 * math.pi * fc / fs
        return math.cos(w0), math.sin(w0), math.sin(w0) / (2.0 * q)

    @staticmethod
    def lowpass(fs, fc, q):
        cs, _, al = Biquad._prelude(fs, fc, q)
        a0 = 1.0 + al
        return Biquad((1 - cs) / 2 / a0, (1 - cs) / a0, (1 - cs) / 2 / a0, -2 * cs / a0, (1 - al) / a0)

    @staticmethod
    def highpass(fs, fc, q):
        cs, _, al = Biquad._prelude(fs, fc, q)
        a0 = 1.0 + al
        return Biquad((1 + cs) / 2 / a0, -(1 + cs) / a0, (1 + cs) / 2 / a0, -2 * cs / a0, (1 - al) / a0)

    @staticmethod
    def bandpass(fs, fc, q):
        cs, sn, al = Biquad._prelude(fs, fc, q)
        a0 = 1.0 + al
        return Biquad(sn / 2 / a0, 0.0, -sn / 2 / a0, -2 * cs / a0, (1 - al) / a0)

    def reset(self):
        self.state = None

    def process_block(self, x):
        y, self.state = _sos_filter(torch.tensor([self.coefficients], dtype=torch.float64), _t(x), self.state)
        return y

    def frequency_response(self, omega):
        b0, b1, b2, a1, a2 = self.coefficients
        z1 = torch.polar(torch.ones(()).double(), -torch.as_tensor(omega, dtype=torch.float64))
        return (b0 + b1 * z1 + b2 * z1 * z1) / (1.0 + a1 * z1 + a2 * z1 * z1)


def butterworth_qs(order: int):
    if order < 2 or order % 2:
        raise ValueError("the order must be even and at least 2 (an odd order needs a first-order section)")
    return [1.0 / (2.0 * math.cos((2 * k - 1) * math.pi / (2 * order))) for k in range(1, order // 2 + 1)]


def chebyshev1_pole_params(order: int, ripple_db: float):
    if order < 2 or order % 2:
        raise ValueError("the order must be even and at least 2")
    eps = math.sqrt(10.0 ** (ripple_db / 10.0) - 1.0)
    a = math.asinh(1.0 / eps) / order
    out = []
    for k in range(1, order // 2 + 1):
        th = (2 * k - 1) * math.pi / (2 * order)
        sigma, omega = math.sinh(a) * math.sin(th), math.cosh(a) * math.cos(th)
        wn = math.hypot(sigma, omega)
        out.append((wn, wn / (2.0 * sigma)))
    return out


class BiquadCascade:
    def __init__(self, stages):
        self.stages = list(stages)
        self.state = None

    def order(self) -> int:
        return 2 * len(self.stages)

    @staticmethod
    def butterworth_lowpass(fs, fc, order):
        return BiquadCascade([Biquad.lowpass(fs, fc, q) for q in butterworth_qs(order)])

    @staticmethod
    def butterworth_highpass(fs, fc, order):
        return BiquadCascade([Biquad.highpass(fs, fc, q) for q in butterworth_qs(order)])

    @staticmethod
    def _warp(fs, fc, wn, highpass):
        """Section corner such that the analogue pole radius ``wn`` lands where the bilinear transform puts it."""
        t = math.tan(math.pi * fc / fs)
        t = t / wn if highpass else t * wn
        return math.atan(t) * fs / math.pi

    @staticmethod
    def chebyshev1_lowpass(fs, fc, order, ripple_db):
        c = BiquadCascade([Biquad.lowpass(fs, BiquadCascade._warp(fs, fc, wn, False), q) for wn, q in chebyshev1_pole_params(order, ripple_db)])
        c.gain = 10.0 ** (-ripple_db / 20.0)                       # even order: the pass band starts at the ripple floor
        return c

    @staticmethod
    def chebyshev1_highpass(fs, fc, order, ripple_db):
        c = BiquadCascade([Biquad.highpass(fs, BiquadCascade._warp(fs, fc, wn, True), q) for wn, q in chebyshev1_pole_params(order, ripple_db)])
        c.gain = 10.0 ** (-ripple_db / 20.0)
        return c

    gain = 1.0

    def reset(self):
        self.state = None

    def sos(self):
        s = torch.tensor([st.coefficients for st in self.stages], dtype=torch.float64)
        if self.gain != 1.0:
            s[0, :3] *= self.gain
        return s

    def process_block(self, x):
        y, self.state = _sos_filter(self.sos(), _t(x), self.state)
        return y

    def frequency_response(self, omega):
        h = torch.as_tensor(self.gain, dtype=torch.complex128)
        for st in self.stages:
            h = h * st.frequency_response(omega)
        return h


def magnitude_db(h):
    return 20.0 * torch.log10(torch.as_tensor(h).abs())


def group_delay(unwrapped_phase, d_omega: float):
    p = _t(unwrapped_phase)
    return -(p[..., 1:] - p[..., :-1]) / d_omega


# ------------------------------------------------------------------ smoothing / resampling
def savgol_coeffs(window_len: int, poly_order: int, deriv: int = 0):
    if window_len < 1 or window_len % 2 == 0:
        raise ValueError("window_len must be odd")
    if not deriv <= poly_order < window_len:
        raise ValueError("need deriv <= poly_order < window_len")
    z = torch.arange(window_len, dtype=torch.float64) - window_len // 2
    a = z[:, None] ** torch.arange(poly_order + 1, dtype=torch.float64)[None, :]
    e = torch.zeros(poly_order + 1, dtype=torch.float64)
    e[deriv] = 1.0
    return math.factorial(deriv) * (a @ torch.linalg.solve(a.t() @ a, e))


def savgol_filter(x, window_len: int, poly_order: int, deriv: int = 0):
    """Correlation with the least-squares coefficients; the edges replicate the first / last sample."""
    x = _t(x)
    c = savgol_coeffs(window_len, poly_order, deriv).to(x.dtype).to(x.device)
    m = window_len // 2
    ext = torch.cat([x[..., :1].expand(*x.shape[:-1], m), x, x[..., -1:].expand(*x.shape[:-1], m)], -1)
    return (ext.unfold(-1, window_len, 1) * c).sum(-1)


def resample_prototype(l: int, m: int, half_taps: int):
    n_taps = 2 * half_taps * l + 1
    k = torch.arange(n_taps, dtype=torch.float64)
    two_fc = 1.0 / max(l, m)
    r = k * (2.0 / (n_taps - 1)) - 1.0
    w = torch.special.i0(6.0 * torch.sqrt((1.0 - r * r).clamp_min(0.0))) / torch.special.i0(torch.tensor(6.0, dtype=torch.float64))
    return l * two_fc * torch.sinc(two_fc * (k - half_taps * l)) * w


def resample(x, l: int, m: int, half_taps: int = 8):
    """Rational rate change by ``l / m`` (zero-stuff, Kaiser-windowed sinc low-pass at 1 / max(l, m), keep every m-th):
    ``len * l // m`` outputs, evaluated polyphase (only the taps that meet a non-zero sample)."""
    if min(l, m, half_taps) < 1:
        raise ValueError("l, m and half_taps must be at least 1")
    x = _t(x)
    h = resample_prototype(l, m, half_taps).to(x.dtype).to(x.device)
    n_out = x.shape[-1] * l // m
    pos = torch.arange(n_out, device=x.device) * m
    k0, p = (pos + l - 1) // l, pos % l
    j = torch.arange(2 * half_taps + 1, device=x.device)
    tap_idx = j[None, :] * l + ((l - p) % l)[:, None]
    taps = torch.where(tap_idx < h.shape[0], h[tap_idx.clamp_max(h.shape[0] - 1)], torch.zeros((), dtype=x.dtype, device=x.device))
    src = k0[:, None] - half_taps + j[None, :]
    ok = (src >= 0) & (src < x.shape[-1])
    return (x[..., src.clamp(0, x.shape[-1] - 1)] * (taps * ok)).sum(-1)


# ------------------------------------------------------------------ wavelets (lifting)
def _haar_fwd(x):
    e, o = x[..., 0::2], x[..., 1::2]
    d = o - e
    return torch.cat([e + d * 0.5, d], -1)


def _haar_inv(x):
    m = x.shape[-1] // 2
    s, d = x[..., :m], x[..., m:]
    e = s - d * 0.5
    return torch.stack([e, d + e], -1).reshape(*x.shape)


def _cdf53_fwd(x):
    e, o = x[..., 0::2], x[..., 1::2]
    d = o - (e + torch.cat([e[..., 1:], e[..., -1:]], -1)) * 0.5
    s = e + (torch.cat([d[..., :1], d[..., :-1]], -1) + d) * 0.25
    return torch.cat([s, d], -1)


def _cdf53_inv(x):
    m = x.shape[-1] // 2
    s, d = x[..., :m], x[..., m:]
    e = s - (torch.cat([d[..., :1], d[..., :-1]], -1) + d) * 0.25
    o = d + (e + torch.cat([e[..., 1:], e[..., -1:]], -1)) * 0.5
    return torch.stack([e, o], -1).reshape(*x.shape)


_WAVELETS = {"haar": (_haar_fwd, _haar_inv), "cdf53": (_cdf53_fwd, _cdf53_inv)}


def dwt_decompose(x, levels: int, wavelet: str = "haar"):
    x = _t(x).clone()
    if x.shape[-1] % (1 << levels):
        raise ValueError(f"length {x.shape[-1]} is not divisible by 2^{levels}")
    for i in range(levels):
        n = x.shape[-1] >> i
        x[..., :n] = _WAVELETS[wavelet][0](x[..., :n])
    return x


def dwt_reconstruct(x, levels: int, wavelet: str = "haar"):
    x = _t(x).clone()
    if x.shape[-1] % (1 << levels):
        raise ValueError(f"length {x.shape[-1]} is not divisible by 2^{levels}")
    for i in reversed(range(levels)):
        n = x.shape[-1] >> i
        x[..., :n] = _WAVELETS[wavelet][1](x[..., :n])
    return x


# ------------------------------------------------------------------ adaptive filters, Kalman, PLL (stateful, sample by sample)
class _Adaptive:
    def __init__(self, n: int):
        self.n = n
        self.reset()

    def reset(self):
        self.weights = torch.zeros(self.n, dtype=torch.float64)
        self.window = torch.zeros(self.n, dtype=torch.float64)          # newest sample first

    def _slide(self, x):
        self.window = torch.cat([torch.tensor([float(x)], dtype=torch.float64), self.window[:-1]])
        return self.window

    def run(self, xs, desired):
        out = [self.update(float(x), float(d)) for x, d in zip(xs, desired)]
        return torch.tensor([o[0] for o in out]), torch.tensor([o[1] for o in out])


class Lms(_Adaptive):
    def __init__(self, n, mu):
        self.mu = mu
        super().__init__(n)

    def update(self, x, desired):
        u = self._slide(x)
        y = float(self.weights @ u)
        err = desired - y
        self.weights = self.weights + self.mu * err * u
        return y, err


class Nlms(_Adaptive):
    def __init__(self, n, mu, eps=1e-8):
        self.mu, self.eps = mu, eps
        super().__init__(n)

    def update(self, x, desired):
        u = self._slide(x)
        y = float(self.weights @ u)
        err = desired - y
        self.weights = self.weights + (self.mu * err / (float(u @ u) + self.eps)) * u
        return y, err


class Rls(_Adaptive):
    def __init__(self, n, lam=0.99, delta=100.0):
        self.lam, self.delta = lam, delta
        super().__init__(n)

    def reset(self):
        super().reset()
        self.p = torch.eye(self.n, dtype=torch.float64) * self.delta

    def update(self, x, desired):
        u = self._slide(x)
        y = float(self.weights @ u)
        err = desired - y
        pu = self.p @ u
        k = pu / (self.lam + float(u @ pu))
        self.weights = self.weights + k * err
        self.p = (self.p - torch.outer(k, pu)) / self.lam
        return y, err


class KalmanFilter:
    """Linear Kalman filter, batched: state ``[..., n]``, covariance ``[..., n, n]`` (Joseph-form update)."""

    def __init__(self, x0, p0):
        self.x, self.p = _t(x0, torch.float64), _t(p0, torch.float64)

    def predict(self, f, q):
        f, q = _t(f, torch.float64), _t(q, torch.float64)
        self.x = (f @ self.x[..., None])[..., 0]
        self.p = f @ self.p @ f.transpose(-1, -2) + q

    def update(self, z, h, r) -> bool:
        z, h, r = _t(z, torch.float64), _t(h, torch.float64), _t(r, torch.float64)
        s = h @ self.p @ h.transpose(-1, -2) + r
        try:
            k = torch.linalg.solve(s, h @ self.p).transpose(-1, -2)
        except RuntimeError:
            return False                                              # singular innovation covariance: state untouched
        self.x = self.x + (k @ (z - (h @ self.x[..., None])[..., 0])[..., None])[..., 0]
        ikh = torch.eye(self.p.shape[-1], dtype=torch.float64) - k @ h
        self.p = ikh @ self.p @ ikh.transpose(-1, -2) + k @ r @ k.transpose(-1, -2)
        return True


class Nco:
    def __init__(self, freq_per_sample: float):
        self.freq, self.phase = freq_per_sample, 0.0

    def set_frequency(self, f):
        self.freq = f

    def tick(self):
        s, c = math.sin(2 * math.pi * self.phase), math.cos(2 * math.pi * self.phase)
        self.phase = (self.phase + self.freq) % 1.0
        return s, c


class PiLoopFilter:
    def __init__(self, kp, ki):
        self.kp, self.ki, self.integrator = kp, ki, 0.0

    @staticmethod
    def design(loop_bandwidth, damping, sample_rate):
        th = (loop_bandwidth / sample_rate) / (damping + 1.0 / (4.0 * damping))
        den = 1.0 + 2.0 * damping * th + th * th
        return PiLoopFilter(4.0 * damping * th / den, 4.0 * th * th / den)

    def reset(self):
        self.integrator = 0.0

    def step(self, e):
        self.integrator += self.ki * e
        return self.kp * e + self.integrator


class Pll:
    """Second-order phase-locked loop on quadrature input: the NCO frequency tracks the tone's."""

    def __init__(self, sample_rate, center_freq, loop_bandwidth, damping=0.7071):
        self.fs, self.center = sample_rate, center_freq / sample_rate
        self.nco, self.filter, self.last_error = Nco(self.center), PiLoopFilter.design(loop_bandwidth, damping, sample_rate), 0.0

    def process_quadrature(self, i, q):
        s, c = self.nco.tick()
        err = math.atan2(q * c - i * s, i * c + q * s) / (2 * math.pi)
        self.last_error = err
        self.nco.set_frequency(self.center + self.filter.step(err))
        return err

    def frequency_estimate(self):
        return self.nco.freq * self.fs

    def locked(self, threshold):
        return abs(self.last_error) < threshold
