"""Audio transforms for ``Dataset.map``: each is a callable on numpy arrays ``[..., time]`` (waveforms) or
``[..., freq, time]`` (spectrograms) returning numpy arrays.  Spectral transforms run on torch's FFT; the IIR
filters use the standard audio-EQ-cookbook biquad coefficients evaluated with ``scipy.signal.lfilter``.

Parity: python/mindspore/dataset/audio/transforms.py, utils.py (the sox / librosa conventions the reference
follows are kept: ``power=2`` spectrograms, HTK or Slaney mel scales, ``top_db`` clamping, mu-law with
``quantization_channels`` levels)."""
from __future__ import annotations

import enum
import math

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------------- enums
class BorderType(str, enum.Enum):
    CONSTANT, EDGE, REFLECT, SYMMETRIC = "constant", "edge", "reflect", "symmetric"


class DensityFunction(str, enum.Enum):
    TPDF, RPDF, GPDF = "TPDF", "RPDF", "GPDF"


class FadeShape(str, enum.Enum):
    QUARTER_SINE, HALF_SINE, LINEAR, LOGARITHMIC, EXPONENTIAL = ("quarter_sine", "half_sine", "linear", "logarithmic",
                                                                 "exponential")


class GainType(str, enum.Enum):
    AMPLITUDE, POWER, DB = "amplitude", "power", "db"


class Interpolation(str, enum.Enum):
    LINEAR, QUADRATIC = "linear", "quadratic"


class MelType(str, enum.Enum):
    HTK, SLANEY = "htk", "slaney"


class Modulation(str, enum.Enum):
    SINUSOIDAL, TRIANGULAR = "sinusoidal", "triangular"


class NormMode(str, enum.Enum):
    NONE, ORTHO = "none", "ortho"


class NormType(str, enum.Enum):
    NONE, SLANEY = "none", "slaney"


class ResampleMethod(str, enum.Enum):
    SINC_INTERPOLATION, KAISER_WINDOW = "sinc_interpolation", "kaiser_window"


class ScaleType(str, enum.Enum):
    MAGNITUDE, POWER = "magnitude", "power"


class WindowType(str, enum.Enum):
    BARTLETT, BLACKMAN, HAMMING, HANN, KAISER = "bartlett", "blackman", "hamming", "hann", "kaiser"


def _val(e):
    return e.value if isinstance(e, enum.Enum) else e


# ---------------------------------------------------------------------------------------------------- helpers
def _hz_to_mel(f, mel_type):
    f = np.asarray(f, dtype=np.float64)
    if _val(mel_type) == "htk":
        return 2595.0 * np.log10(1.0 + f / 700.0)
    lin = f / (200.0 / 3)
    log_part = 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (math.log(6.4) / 27.0)
    return np.where(f >= 1000.0, log_part, lin)


def _mel_to_hz(m, mel_type):
    m = np.asarray(m, dtype=np.float64)
    if _val(mel_type) == "htk":
        return 700.0 * (10.0 ** (m / 2595.0) - 1.0)
    return np.where(m >= 15.0, 1000.0 * np.exp((math.log(6.4) / 27.0) * (m - 15.0)), m * (200.0 / 3))


def melscale_fbanks(n_freqs, f_min, f_max, n_mels, sample_rate, norm=NormType.NONE, mel_type=MelType.HTK):
    """Triangular mel filter bank [n_freqs, n_mels]."""
    freqs = np.linspace(0, sample_rate // 2, n_freqs)
    pts = _mel_to_hz(np.linspace(_hz_to_mel(f_min, mel_type), _hz_to_mel(f_max, mel_type), n_mels + 2), mel_type)
    diff = pts[1:] - pts[:-1]
    slopes = pts[None, :] - freqs[:, None]
    down = -slopes[:, :-2] / diff[:-1]
    up = slopes[:, 2:] / diff[1:]
    fb = np.maximum(0.0, np.minimum(down, up))
    if _val(norm) == "slaney":
        fb = fb * (2.0 / (pts[2:n_mels + 2] - pts[:n_mels]))[None, :]
    return fb.astype(np.float32)


def linear_fbanks(n_freqs, f_min, f_max, n_filter, sample_rate):
    freqs = np.linspace(0, sample_rate // 2, n_freqs)
    pts = np.linspace(f_min, f_max, n_filter + 2)
    diff = pts[1:] - pts[:-1]
    slopes = pts[None, :] - freqs[:, None]
    return np.maximum(0.0, np.minimum(-slopes[:, :-2] / diff[:-1], slopes[:, 2:] / diff[1:])).astype(np.float32)


def create_dct(n_mfcc, n_mels, norm=NormMode.NONE):
    """DCT-II matrix [n_mels, n_mfcc]."""
    n = np.arange(n_mels, dtype=np.float64)
    k = np.arange(n_mfcc, dtype=np.float64)[:, None]
    dct = np.cos(math.pi / n_mels * (n + 0.5) * k)
    if _val(norm) == "ortho":
        dct[0] *= 1.0 / math.sqrt(2.0)
        dct *= math.sqrt(2.0 / n_mels)
    else:
        dct *= 2.0
    return dct.T.astype(np.float32)


def _window(kind, n):
    kind = _val(kind)
    fn = {"hann": torch.hann_window, "hamming": torch.hamming_window, "blackman": torch.blackman_window,
          "bartlett": torch.bartlett_window, "kaiser": torch.kaiser_window}[kind]
    return fn(n, periodic=True)


def _t(x):
    return torch.as_tensor(np.ascontiguousarray(x))


class AudioTensorOperation:
    """Base of the audio transforms: ``op(waveform)`` with numpy (or anything ``np.asarray`` takes) in and out."""

    def __call__(self, *inputs):
        out = self._run(*[np.asarray(i) for i in inputs])
        return out

    def _run(self, x):
        raise NotImplementedError


# ---------------------------------------------------------------------------------------------------- filters
class Biquad(AudioTensorOperation):
    """y[n] = (b0 x[n] + b1 x[n-1] + b2 x[n-2] - a1 y[n-1] - a2 y[n-2]) / a0, clamped to [-1, 1]."""

    def __init__(self, b0, b1, b2, a0, a1, a2):
        if a0 == 0:
            raise ValueError("Biquad: a0 must not be 0")
        self.b, self.a = [b0, b1, b2], [a0, a1, a2]

    def _run(self, x):
        import scipy.signal
        y = scipy.signal.lfilter(np.asarray(self.b) / self.a[0], np.asarray(self.a) / self.a[0], x.astype(np.float64))
        return np.clip(y, -1.0, 1.0).astype(x.dtype if x.dtype.kind == "f" else np.float32)


def _cookbook(kind):
    def coeffs(sr, f0, q, gain=0.0, const_skirt=False, noise=False):
        w0 = 2 * math.pi * f0 / sr
        alpha = math.sin(w0) / (2 * q)
        cw = math.cos(w0)
        a = 10 ** (gain / 40.0)
        if kind == "lowpass":
            return ((1 - cw) / 2, 1 - cw, (1 - cw) / 2, 1 + alpha, -2 * cw, 1 - alpha)
        if kind == "highpass":
            return ((1 + cw) / 2, -1 - cw, (1 + cw) / 2, 1 + alpha, -2 * cw, 1 - alpha)
        if kind == "bandpass":
            t = math.sin(w0) / 2 if const_skirt else alpha
            return (t, 0.0, -t, 1 + alpha, -2 * cw, 1 - alpha)
        if kind == "bandreject":
            return (1.0, -2 * cw, 1.0, 1 + alpha, -2 * cw, 1 - alpha)
        if kind == "allpass":
            return (1 - alpha, -2 * cw, 1 + alpha, 1 + alpha, -2 * cw, 1 - alpha)
        if kind == "equalizer":
            return (1 + alpha * a, -2 * cw, 1 - alpha * a, 1 + alpha / a, -2 * cw, 1 - alpha / a)
        sq = 2 * math.sqrt(a) * alpha
        if kind == "bass":
            return (a * ((a + 1) - (a - 1) * cw + sq), 2 * a * ((a - 1) - (a + 1) * cw), a * ((a + 1) - (a - 1) * cw - sq),
                    (a + 1) + (a - 1) * cw + sq, -2 * ((a - 1) + (a + 1) * cw), (a + 1) + (a - 1) * cw - sq)
        if kind == "treble":
            return (a * ((a + 1) + (a - 1) * cw + sq), -2 * a * ((a - 1) + (a + 1) * cw),
                    a * ((a + 1) + (a - 1) * cw - sq), (a + 1) - (a - 1) * cw + sq, 2 * ((a - 1) - (a + 1) * cw),
                    (a + 1) - (a - 1) * cw - sq)
        raise ValueError(kind)
    return coeffs


def _biquad_class(name, kind, params, doc):
    def __init__(self, sample_rate, *args, **kwargs):
        vals = dict(params)
        for (k, _), v in zip(params, args):
            vals[k] = v
        vals.update(kwargs)
        if sample_rate == 0:
            raise ValueError("%s: sample_rate must not be 0" % name)
        q = vals.get("Q", 0.707)
        if not 0 < q <= 1 and kind not in ("equalizer",):
            raise ValueError("%s: Q must be in (0, 1], but got %r" % (name, q))
        f0 = vals.get("cutoff_freq", vals.get("central_freq", vals.get("center_freq", 1000.0)))
        Biquad.__init__(self, *_cookbook(kind)(sample_rate, f0, q, vals.get("gain", 0.0),
                                               vals.get("const_skirt_gain", False), vals.get("noise", False)))
    return type(name, (Biquad,), {"__init__": __init__, "__doc__": doc})


LowpassBiquad = _biquad_class("LowpassBiquad", "lowpass", [("cutoff_freq", 1000.0), ("Q", 0.707)],
                              "Two-pole low-pass at ``cutoff_freq``.")
HighpassBiquad = _biquad_class("HighpassBiquad", "highpass", [("cutoff_freq", 1000.0), ("Q", 0.707)],
                               "Two-pole high-pass at ``cutoff_freq``.")
BandpassBiquad = _biquad_class("BandpassBiquad", "bandpass", [("central_freq", 1000.0), ("Q", 0.707),
                                                              ("const_skirt_gain", False)], "Two-pole band-pass.")
BandrejectBiquad = _biquad_class("BandrejectBiquad", "bandreject", [("central_freq", 1000.0), ("Q", 0.707)],
                                 "Two-pole band-reject (notch).")
AllpassBiquad = _biquad_class("AllpassBiquad", "allpass", [("central_freq", 1000.0), ("Q", 0.707)],
                              "Two-pole all-pass.")
EqualizerBiquad = _biquad_class("EqualizerBiquad", "equalizer", [("center_freq", 1000.0), ("gain", 0.0),
                                                                 ("Q", 0.707)], "Peaking equaliser.")
BassBiquad = _biquad_class("BassBiquad", "bass", [("gain", 0.0), ("central_freq", 100.0), ("Q", 0.707)],
                           "Low-shelf tone control.")
TrebleBiquad = _biquad_class("TrebleBiquad", "treble", [("gain", 0.0), ("central_freq", 3000.0), ("Q", 0.707)],
                             "High-shelf tone control.")


class BandBiquad(Biquad):
    """Two-pole band-pass in sox's ``band`` form (``noise=True`` for unpitched audio)."""

    def __init__(self, sample_rate, central_freq, Q=0.707, noise=False):  # noqa: N803
        w0 = 2 * math.pi * central_freq / sample_rate
        bw = w0 / Q
        a2 = math.exp(-bw)
        a1 = -4 * a2 / (1 + a2) * math.cos(w0)
        b0 = math.sqrt(1 - a1 * a1 / (4 * a2)) * (1 - a2)
        if noise:
            b0 *= math.sqrt(((1 + a2) ** 2 - a1 * a1) * (1 - a2) / (1 + a2)) / b0
        super().__init__(b0, 0.0, 0.0, 1.0, a1, a2)


class DeemphBiquad(Biquad):
    """CD de-emphasis (a high-shelf of about -9.5 dB) for 44.1 or 48 kHz audio."""

    def __init__(self, sample_rate):
        if sample_rate not in (44100, 48000):
            raise ValueError("DeemphBiquad: sample_rate must be 44100 or 48000, but got %r" % (sample_rate,))
        f0, slope, gain = (5283.0, 0.4845, -9.477) if sample_rate == 44100 else (5356.0, 0.479, -9.62)
        w0 = 2 * math.pi * f0 / sample_rate
        a = 10 ** (gain / 40.0)
        alpha = math.sin(w0) / 2 * math.sqrt((a + 1 / a) * (1 / slope - 1) + 2)
        cw, sq = math.cos(w0), 2 * math.sqrt(a) * alpha
        super().__init__(a * ((a + 1) + (a - 1) * cw + sq), -2 * a * ((a - 1) + (a + 1) * cw),
                         a * ((a + 1) + (a - 1) * cw - sq), (a + 1) - (a - 1) * cw + sq,
                         2 * ((a - 1) - (a + 1) * cw), (a + 1) - (a - 1) * cw - sq)


class RiaaBiquad(AudioTensorOperation):
    """RIAA vinyl playback equalisation (44.1, 48, 88.2 or 96 kHz)."""
    _ZEROS = {44100: [-0.2014898, 0.9233820], 48000: [-0.1766069, 0.9321590], 88200: [-0.1168735, 0.9648312],
              96000: [-0.1141486, 0.9676817]}
    _POLES = {44100: [0.7083149, 0.9924091], 48000: [0.7396325, 0.9931330], 88200: [0.8590646, 0.9964002],
              96000: [0.8699137, 0.9966946]}

    def __init__(self, sample_rate):
        if sample_rate not in self._ZEROS:
            raise ValueError("RiaaBiquad: sample_rate must be one of %s" % sorted(self._ZEROS))
        z, p = self._ZEROS[sample_rate], self._POLES[sample_rate]
        b = np.array([1.0, -(z[0] + z[1]), z[0] * z[1]])
        a = np.array([1.0, -(p[0] + p[1]), p[0] * p[1]])
        w = 2 * math.pi * 1000.0 / sample_rate                       # unit gain at 1 kHz
        ej = np.exp(-1j * w * np.arange(3))
        self.b, self.a = b / abs((b * ej).sum() / (a * ej).sum()), a

    def _run(self, x):
        import scipy.signal
        return np.clip(scipy.signal.lfilter(self.b, self.a, x.astype(np.float64)), -1, 1).astype(np.float32)


class LFilter(AudioTensorOperation):
    """IIR filter with denominator ``a_coeffs`` and numerator ``b_coeffs`` (lowest delay first)."""

    def __init__(self, a_coeffs, b_coeffs, clamp=True):
        if len(a_coeffs) != len(b_coeffs):
            raise ValueError("LFilter: a_coeffs and b_coeffs must have the same length")
        if a_coeffs[0] == 0:
            raise ValueError("LFilter: a_coeffs[0] must not be 0")
        self.a, self.b, self.clamp = np.asarray(a_coeffs, float), np.asarray(b_coeffs, float), clamp

    def _run(self, x):
        import scipy.signal
        y = scipy.signal.lfilter(self.b / self.a[0], self.a / self.a[0], x.astype(np.float64))
        return (np.clip(y, -1, 1) if self.clamp else y).astype(np.float32)


class Filtfilt(LFilter):
    """The filter applied forward, then backward (zero phase)."""

    def _run(self, x):
        import scipy.signal
        f = lambda v: scipy.signal.lfilter(self.b / self.a[0], self.a / self.a[0], v)
        y = f(f(x.astype(np.float64))[..., ::-1])[..., ::-1]
        return (np.clip(y, -1, 1) if self.clamp else y).astype(np.float32)


# ---------------------------------------------------------------------------------------------------- level / shape
class AmplitudeToDB(AudioTensorOperation):
    def __init__(self, stype=ScaleType.POWER, ref_value=1.0, amin=1e-10, top_db=80.0):
        if amin <= 0 or ref_value <= 0 or (top_db is not None and top_db <= 0):
            raise ValueError("AmplitudeToDB: amin, ref_value and top_db must be positive")
        self.mult = 10.0 if _val(stype) == "power" else 20.0
        self.ref, self.amin, self.top_db = ref_value, amin, top_db

    def _run(self, x):
        db = self.mult * (np.log10(np.maximum(x, self.amin)) - math.log10(max(self.amin, self.ref)))
        if self.top_db is not None:
            peak = db.reshape(db.shape[:-3] + (-1,)).max(-1).reshape(db.shape[:-3] + (1, 1, 1)) if db.ndim >= 3 \
                else db.max()
            db = np.maximum(db, peak - self.top_db)
        return db.astype(np.float32)


class DBToAmplitude(AudioTensorOperation):
    def __init__(self, ref, power):
        self.ref, self.power = ref, power

    def _run(self, x):
        return (self.ref * np.power(np.power(10.0, 0.1 * x), self.power)).astype(np.float32)


class Angle(AudioTensorOperation):
    """Phase of ``[..., 2]`` (real, imaginary) input."""

    def _run(self, x):
        return np.arctan2(x[..., 1], x[..., 0]).astype(x.dtype)


class ComplexNorm(AudioTensorOperation):
    def __init__(self, power=1.0):
        if power < 0:
            raise ValueError("ComplexNorm: power must be non-negative")
        self.power = power

    def _run(self, x):
        return np.power(x[..., 0] ** 2 + x[..., 1] ** 2, 0.5 * self.power).astype(x.dtype)


class Magphase(AudioTensorOperation):
    def __init__(self, power=1.0):
        self.power = power

    def _run(self, x):
        return ComplexNorm(self.power)._run(x), Angle()._run(x)


class Contrast(AudioTensorOperation):
    """sox ``contrast``: x -> sin(x pi/2 + c sin(4 x pi/2)) with c = enhancement_amount / 750."""

    def __init__(self, enhancement_amount=75.0):
        if not 0 <= enhancement_amount <= 100:
            raise ValueError("Contrast: enhancement_amount must be in [0, 100]")
        self.c = enhancement_amount / 750.0

    def _run(self, x):
        t = x * (math.pi / 2)
        return np.sin(t + self.c * np.sin(t * 4)).astype(np.float32)


class DCShift(AudioTensorOperation):
    def __init__(self, shift, limiter_gain=None):
        if not -2.0 <= shift <= 2.0:
            raise ValueError("DCShift: shift must be in [-2, 2]")
        self.shift, self.limiter = shift, limiter_gain

    def _run(self, x):
        if self.limiter is None:
            return np.clip(x + self.shift, -1, 1).astype(np.float32)
        thr = 1.0 - (abs(self.shift) - self.limiter)
        y = x + self.shift
        if self.shift > 0:
            hi = x > thr
            y = np.where(hi, (x - thr) * self.limiter / (1 - thr) + thr + self.shift, y)
        elif self.shift < 0:
            lo = x < -thr
            y = np.where(lo, (x + thr) * self.limiter / (1 - thr) - thr + self.shift, y)
        return np.clip(y, -1, 1).astype(np.float32)


class Dither(AudioTensorOperation):
    """Adds noise of one 16-bit step before rounding to 16 bits (TPDF: triangular, RPDF: uniform, GPDF: normal)."""

    def __init__(self, density_function=DensityFunction.TPDF, noise_shaping=False):
        self.kind, self.shaping = _val(density_function), noise_shaping

    def _run(self, x):
        rng = np.random.default_rng()
        scale = 2.0 ** 15
        if self.kind == "RPDF":
            noise = rng.uniform(-0.5, 0.5, x.shape)
        elif self.kind == "GPDF":
            noise = rng.normal(0, 0.5, x.shape)
        else:
            noise = rng.uniform(-0.5, 0.5, x.shape) + rng.uniform(-0.5, 0.5, x.shape)
        return (np.round(x * scale + noise) / scale).astype(np.float32)


class Fade(AudioTensorOperation):
    def __init__(self, fade_in_len=0, fade_out_len=0, fade_shape=FadeShape.LINEAR):
        if fade_in_len < 0 or fade_out_len < 0:
            raise ValueError("Fade: lengths must be non-negative")
        self.n_in, self.n_out, self.shape = fade_in_len, fade_out_len, _val(fade_shape)

    def _curve(self, n):
        t = np.linspace(0, 1, n)
        return {"linear": t, "exponential": np.power(2.0, t - 1) * t, "logarithmic": np.log10(0.1 + t) + 1,
                "quarter_sine": np.sin(t * math.pi / 2), "half_sine": np.sin(t * math.pi - math.pi / 2) / 2 + 0.5}[
            self.shape]

    def _run(self, x):
        n = x.shape[-1]
        if self.n_in > n or self.n_out > n:
            raise ValueError("Fade: the fade lengths exceed the waveform length %d" % n)
        env = np.ones(n)
        if self.n_in:
            env[:self.n_in] = np.clip(self._curve(self.n_in), 0, 1)
        if self.n_out:
            env[n - self.n_out:] *= np.clip(self._curve(self.n_out)[::-1], 0, 1)
        return (x * env).astype(np.float32)


class Gain(AudioTensorOperation):
    def __init__(self, gain_db=1.0):
        self.ratio = 10 ** (gain_db / 20.0)

    def _run(self, x):
        return (x * self.ratio).astype(np.float32)


class Vol(AudioTensorOperation):
    def __init__(self, gain, gain_type=GainType.AMPLITUDE):
        kind = _val(gain_type)
        if kind in ("amplitude", "power") and gain < 0:
            raise ValueError("Vol: gain must be non-negative for %s" % kind)
        self.ratio = gain if kind == "amplitude" else math.sqrt(gain) if kind == "power" else 10 ** (gain / 20.0)

    def _run(self, x):
        return np.clip(x * self.ratio, -1, 1).astype(np.float32)


class Overdrive(AudioTensorOperation):
    """sox ``overdrive``: soft clipping of the boosted signal with a one-pole DC blocker."""

    def __init__(self, gain=20.0, color=20.0):
        if not 0 <= gain <= 100 or not 0 <= color <= 100:
            raise ValueError("Overdrive: gain and color must be in [0, 100]")
        self.gain, self.color = 10 ** (gain / 20.0), color / 200.0

    def _run(self, x):
        t = x.astype(np.float64) * self.gain + self.color
        t = np.clip(t, -1, 1)
        t = t - t ** 3 / 3.0
        out = np.zeros_like(t)
        last_in = np.zeros(t.shape[:-1])
        last_out = np.zeros(t.shape[:-1])
        for i in range(t.shape[-1]):
            last_out = t[..., i] - last_in + 0.995 * last_out
            last_in = t[..., i]
            out[..., i] = x[..., i] * 0.5 + last_out * 0.75
        return np.clip(out, -1, 1).astype(np.float32)


class MuLawEncoding(AudioTensorOperation):
    def __init__(self, quantization_channels=256):
        if quantization_channels <= 0:
            raise ValueError("MuLawEncoding: quantization_channels must be positive")
        self.mu = quantization_channels - 1.0

    def _run(self, x):
        y = np.sign(x) * np.log1p(self.mu * np.abs(x)) / math.log1p(self.mu)
        return ((y + 1) / 2 * self.mu + 0.5).astype(np.int32)


class MuLawDecoding(AudioTensorOperation):
    def __init__(self, quantization_channels=256):
        self.mu = quantization_channels - 1.0

    def _run(self, x):
        y = x.astype(np.float64) / self.mu * 2 - 1.0
        return (np.sign(y) * (np.exp(np.abs(y) * math.log1p(self.mu)) - 1.0) / self.mu).astype(np.float32)


class ComputeDeltas(AudioTensorOperation):
    """Delta coefficients along time over a window of ``win_length`` frames."""

    def __init__(self, win_length=5, pad_mode=BorderType.EDGE):
        if win_length < 3:
            raise ValueError("ComputeDeltas: win_length must be at least 3")
        self.n, self.mode = (win_length - 1) // 2, _val(pad_mode)

    def _run(self, x):
        n = self.n
        pad = [(0, 0)] * (x.ndim - 1) + [(n, n)]
        p = np.pad(x.astype(np.float64), pad, mode=self.mode)
        k = np.arange(-n, n + 1, dtype=np.float64)
        out = sum(k[j] * p[..., j:j + x.shape[-1]] for j in range(2 * n + 1)) / (2 * (np.arange(1, n + 1) ** 2).sum())
        return out.astype(np.float32)


class SlidingWindowCmn(AudioTensorOperation):
    """Cepstral mean (and optionally variance) normalisation over a sliding window of frames, input
    [..., time, freq]."""

    def __init__(self, cmn_window=600, min_cmn_window=100, center=False, norm_vars=False):
        self.w, self.min_w, self.center, self.norm_vars = cmn_window, min_cmn_window, center, norm_vars

    def _run(self, x):
        t = x.shape[-2]
        out = np.empty_like(x, dtype=np.float32)
        for i in range(t):
            if self.center:
                lo, hi = i - self.w // 2, i - self.w // 2 + self.w
            else:
                lo, hi = i - self.w, i + 1
            if lo < 0:
                hi, lo = hi - lo, 0
            if not self.center and hi > i + 1:
                hi = max(i + 1, self.min_w)
            if hi > t:
                lo, hi = max(0, lo - (hi - t)), t
            win = x[..., lo:hi, :]
            out[..., i, :] = x[..., i, :] - win.mean(-2)
            if self.norm_vars:
                out[..., i, :] /= np.sqrt(np.maximum(win.var(-2), 1e-20))
        return out


# ---------------------------------------------------------------------------------------------------- spectral
class Spectrogram(AudioTensorOperation):
    def __init__(self, n_fft=400, win_length=None, hop_length=None, pad=0, window=WindowType.HANN, power=2.0,
                 normalized=False, center=True, pad_mode=BorderType.REFLECT, onesided=True):
        self.n_fft, self.win = n_fft, win_length or n_fft
        self.hop = hop_length or self.win // 2
        if self.win > n_fft:
            raise ValueError("Spectrogram: win_length must not exceed n_fft")
        self.pad, self.window, self.power, self.normalized = pad, window, power, normalized
        self.center, self.pad_mode, self.onesided = center, _val(pad_mode), onesided

    def _stft(self, x):
        t = _t(x).float()
        if self.pad:
            t = torch.nn.functional.pad(t, (self.pad, self.pad))
        lead = t.shape[:-1]
        mode = {"edge": "replicate", "symmetric": "reflect"}.get(self.pad_mode, self.pad_mode)
        spec = torch.stft(t.reshape(-1, t.shape[-1]), self.n_fft, self.hop, self.win, _window(self.window, self.win),
                          self.center, mode, False, self.onesided, return_complex=True)
        if self.normalized:
            spec = spec / _window(self.window, self.win).pow(2).sum().sqrt()
        return spec.reshape(lead + spec.shape[-2:])

    def _run(self, x):
        spec = self._stft(x)
        if self.power is None or self.power == 0:
            return torch.view_as_real(spec).numpy()
        return spec.abs().pow(self.power).numpy().astype(np.float32)


class InverseSpectrogram(AudioTensorOperation):
    """Waveform from a complex spectrogram given as [..., freq, time, 2]."""

    def __init__(self, length=None, n_fft=400, win_length=None, hop_length=None, pad=0, window=WindowType.HANN,
                 normalized=False, center=True, pad_mode=BorderType.REFLECT, onesided=True):
        self.length, self.n_fft, self.win = length, n_fft, win_length or n_fft
        self.hop = hop_length or self.win // 2
        self.pad, self.window, self.normalized, self.center, self.onesided = pad, window, normalized, center, onesided

    def _run(self, x):
        spec = torch.view_as_complex(_t(x).float().contiguous())
        if self.normalized:
            spec = spec * _window(self.window, self.win).pow(2).sum().sqrt()
        lead = spec.shape[:-2]
        wav = torch.istft(spec.reshape((-1,) + spec.shape[-2:]), self.n_fft, self.hop, self.win,
                          _window(self.window, self.win), self.center, False, self.onesided,
                          self.length + 2 * self.pad if self.length else None)
        if self.pad:
            wav = wav[..., self.pad:wav.shape[-1] - self.pad]
        return wav.reshape(lead + wav.shape[-1:]).numpy()


class GriffinLim(AudioTensorOperation):
    """Phase reconstruction of a magnitude / power spectrogram by iterated STFT consistency."""

    def __init__(self, n_fft=400, n_iter=32, win_length=None, hop_length=None, window_type=WindowType.HANN, power=2.0,
                 momentum=0.99, length=None, rand_init=True):
        if not 0 <= momentum < 1:
            raise ValueError("GriffinLim: momentum must be in [0, 1)")
        self.n_fft, self.n_iter, self.win = n_fft, n_iter, win_length or n_fft
        self.hop = hop_length or self.win // 2
        self.window, self.power, self.momentum, self.length, self.rand = window_type, power, momentum, length, rand_init

    def _run(self, x):
        mag = _t(x).float().pow(1.0 / self.power)
        lead = mag.shape[:-2]
        mag = mag.reshape((-1,) + mag.shape[-2:])
        w = _window(self.window, self.win)
        angles = torch.exp(2j * math.pi * torch.rand(mag.shape)) if self.rand else torch.ones(mag.shape,
                                                                                               dtype=torch.complex64)
        prev = torch.zeros_like(angles)
        m = self.momentum / (1 + self.momentum)
        for _ in range(self.n_iter):
            wav = torch.istft(mag * angles, self.n_fft, self.hop, self.win, w, length=self.length)
            rebuilt = torch.stft(wav, self.n_fft, self.hop, self.win, w, True, "reflect", False, True,
                                 return_complex=True)
            angles = rebuilt - prev * m
            angles = angles / (angles.abs() + 1e-16)
            prev = rebuilt
        wav = torch.istft(mag * angles, self.n_fft, self.hop, self.win, w, length=self.length)
        return wav.reshape(lead + wav.shape[-1:]).numpy()


class MelScale(AudioTensorOperation):
    def __init__(self, n_mels=128, sample_rate=16000, f_min=0.0, f_max=None, n_stft=201, norm=NormType.NONE,
                 mel_type=MelType.HTK):
        f_max = f_max if f_max is not None else sample_rate // 2
        if f_min > f_max:
            raise ValueError("MelScale: f_min must not exceed f_max")
        self.fb = melscale_fbanks(n_stft, f_min, f_max, n_mels, sample_rate, norm, mel_type)

    def _run(self, x):
        return np.einsum("...ft,fm->...mt", x.astype(np.float32), self.fb)


class InverseMelScale(AudioTensorOperation):
    """Least-squares estimate (non-negative) of the linear-frequency spectrogram behind a mel spectrogram."""

    def __init__(self, n_stft, n_mels=128, sample_rate=16000, f_min=0.0, f_max=None, max_iter=100000,
                 tolerance_loss=1e-5, tolerance_change=1e-8, sgdargs=None, norm=NormType.NONE, mel_type=MelType.HTK):
        f_max = f_max if f_max is not None else sample_rate // 2
        self.fb = melscale_fbanks(n_stft, f_min, f_max, n_mels, sample_rate, norm, mel_type)

    def _run(self, x):
        pinv = np.linalg.pinv(self.fb.T.astype(np.float64))                   # [n_stft, n_mels]
        return np.maximum(np.einsum("fm,...mt->...ft", pinv, x.astype(np.float64)), 0).astype(np.float32)


class MelSpectrogram(AudioTensorOperation):
    def __init__(self, sample_rate=16000, n_fft=400, win_length=None, hop_length=None, f_min=0.0, f_max=None, pad=0,
                 n_mels=128, window=WindowType.HANN, power=2.0, normalized=False, center=True,
                 pad_mode=BorderType.REFLECT, onesided=True, norm=NormType.NONE, mel_scale=MelType.HTK):
        self.spec = Spectrogram(n_fft, win_length, hop_length, pad, window, power, normalized, center, pad_mode,
                                onesided)
        self.mel = MelScale(n_mels, sample_rate, f_min, f_max, n_fft // 2 + 1, norm, mel_scale)

    def _run(self, x):
        return self.mel._run(self.spec._run(x))


class MFCC(AudioTensorOperation):
    def __init__(self, sample_rate=16000, n_mfcc=40, dct_type=2, norm=NormMode.ORTHO, log_mels=False,
                 melkwargs=None):
        if dct_type != 2:
            raise ValueError("MFCC: only dct_type 2 is supported")
        kw = dict(melkwargs or {})
        self.mel = MelSpectrogram(sample_rate, kw.get("n_fft", 400), kw.get("win_length"), kw.get("hop_length"),
                                  kw.get("f_min", 0.0), kw.get("f_max"), kw.get("pad", 0), kw.get("n_mels", 128),
                                  kw.get("window", WindowType.HANN), kw.get("power", 2.0),
                                  kw.get("normalized", False), kw.get("center", True),
                                  kw.get("pad_mode", BorderType.REFLECT), kw.get("onesided", True),
                                  kw.get("norm", NormType.NONE), kw.get("mel_scale", MelType.HTK))
        n_mels = kw.get("n_mels", 128)
        if n_mfcc > n_mels:
            raise ValueError("MFCC: n_mfcc must not exceed n_mels")
        self.dct, self.log_mels = create_dct(n_mfcc, n_mels, norm), log_mels
        self.to_db = AmplitudeToDB(ScaleType.POWER, 1.0, 1e-10, 80.0)

    def _run(self, x):
        mel = self.mel._run(x)
        mel = np.log(mel + 1e-6) if self.log_mels else self.to_db._run(mel)
        return np.einsum("...mt,mk->...kt", mel, self.dct).astype(np.float32)


class LFCC(AudioTensorOperation):
    def __init__(self, sample_rate=16000, n_filter=128, n_lfcc=40, f_min=0.0, f_max=None, dct_type=2,
                 norm=NormMode.ORTHO, log_lf=False, speckwargs=None):
        kw = dict(speckwargs or {})
        n_fft = kw.get("n_fft", 400)
        self.spec = Spectrogram(n_fft, kw.get("win_length"), kw.get("hop_length"), kw.get("pad", 0),
                                kw.get("window", WindowType.HANN), kw.get("power", 2.0), kw.get("normalized", False),
                                kw.get("center", True), kw.get("pad_mode", BorderType.REFLECT),
                                kw.get("onesided", True))
        self.fb = linear_fbanks(n_fft // 2 + 1, f_min, f_max if f_max is not None else sample_rate // 2, n_filter,
                                sample_rate)
        self.dct, self.log_lf = create_dct(n_lfcc, n_filter, norm), log_lf
        self.to_db = AmplitudeToDB(ScaleType.POWER, 1.0, 1e-10, 80.0)

    def _run(self, x):
        lin = np.einsum("...ft,fm->...mt", self.spec._run(x), self.fb)
        lin = np.log(lin + 1e-6) if self.log_lf else self.to_db._run(lin)
        return np.einsum("...mt,mk->...kt", lin, self.dct).astype(np.float32)


class SpectralCentroid(AudioTensorOperation):
    def __init__(self, sample_rate, n_fft=400, win_length=None, hop_length=None, pad=0, window=WindowType.HANN):
        self.spec = Spectrogram(n_fft, win_length, hop_length, pad, window, 1.0)
        self.freqs = np.linspace(0, sample_rate // 2, n_fft // 2 + 1, dtype=np.float32)

    def _run(self, x):
        s = self.spec._run(x)
        return ((self.freqs[:, None] * s).sum(-2) / np.maximum(s.sum(-2), 1e-20)).astype(np.float32)


class _Mask(AudioTensorOperation):
    axis = -1

    def __init__(self, iid_masks=False, mask_param=0, mask_start=0, mask_value=0.0):
        if mask_param < 0 or mask_start < 0:
            raise ValueError("%s: the mask parameters must be non-negative" % type(self).__name__)
        self.iid, self.param, self.start, self.value = iid_masks, mask_param, mask_start, mask_value

    def _run(self, x):
        out = x.astype(np.float32).copy()
        size = out.shape[self.axis]
        if self.param > size:
            raise ValueError("%s: the mask width %d exceeds the axis length %d" % (type(self).__name__, self.param,
                                                                                     size))
        rng = np.random.default_rng()

        def one(arr):
            width = int(rng.integers(0, self.param + 1))
            start = int(rng.integers(0, size - width + 1)) if self.iid else min(self.start, size - width)
            idx = [slice(None)] * arr.ndim
            idx[self.axis] = slice(start, start + width)
            arr[tuple(idx)] = self.value
        if self.iid and out.ndim > 2:
            for i in range(out.shape[0]):
                one(out[i])
        else:
            one(out)
        return out


class TimeMasking(_Mask):
    axis = -1

    def __init__(self, iid_masks=False, time_mask_param=0, mask_start=0, mask_value=0.0):
        super().__init__(iid_masks, time_mask_param, mask_start, mask_value)


class FrequencyMasking(_Mask):
    axis = -2

    def __init__(self, iid_masks=False, freq_mask_param=0, mask_start=0, mask_value=0.0):
        super().__init__(iid_masks, freq_mask_param, mask_start, mask_value)


class MaskAlongAxis(AudioTensorOperation):
    """Sets ``mask_width`` entries from ``mask_start`` on along ``axis`` (1 = frequency, 2 = time) to ``mask_value``."""

    def __init__(self, mask_start, mask_width, mask_value, axis):
        if axis not in (1, 2):
            raise ValueError("MaskAlongAxis: axis must be 1 (frequency) or 2 (time)")
        self.start, self.width, self.value, self.axis = mask_start, mask_width, mask_value, axis - 3

    def _run(self, x):
        out = x.astype(np.float32).copy()
        idx = [slice(None)] * out.ndim
        idx[self.axis] = slice(self.start, self.start + self.width)
        out[tuple(idx)] = self.value
        return out


class MaskAlongAxisIID(AudioTensorOperation):
    """A random mask of up to ``mask_param`` entries along ``axis``, drawn independently per leading index."""

    def __init__(self, mask_param, mask_value, axis):
        if axis not in (1, 2):
            raise ValueError("MaskAlongAxisIID: axis must be 1 (frequency) or 2 (time)")
        self.param, self.value, self.axis = mask_param, mask_value, axis - 3

    def _run(self, x):
        out = x.astype(np.float32).copy()
        flat = out.reshape((-1,) + out.shape[-2:])
        rng = np.random.default_rng()
        size = flat.shape[self.axis]
        for i in range(flat.shape[0]):
            width = rng.uniform(0, self.param)
            start = rng.uniform(0, size - width)
            idx = [i, slice(None), slice(None)]
            idx[self.axis + 3] = slice(int(start), int(start + width))
            flat[tuple(idx)] = self.value
        return flat.reshape(out.shape)


class PhaseVocoder(AudioTensorOperation):
    """Time-stretches a complex spectrogram [..., freq, time, 2] by ``rate`` without changing pitch."""

    def __init__(self, rate, phase_advance):
        if rate <= 0:
            raise ValueError("PhaseVocoder: rate must be positive")
        self.rate, self.adv = rate, np.asarray(phase_advance, dtype=np.float64)

    def _run(self, x):
        spec = x[..., 0].astype(np.float64) + 1j * x[..., 1].astype(np.float64)
        steps = np.arange(0, spec.shape[-1], self.rate)
        spec = np.pad(spec, [(0, 0)] * (spec.ndim - 1) + [(0, 2)])
        i0 = steps.astype(int)
        a0, a1 = spec[..., i0], spec[..., i0 + 1]
        alpha = steps % 1.0
        mag = alpha * np.abs(a1) + (1 - alpha) * np.abs(a0)
        phase = np.angle(a1) - np.angle(a0) - self.adv.reshape(-1, 1)
        phase = phase - 2 * math.pi * np.round(phase / (2 * math.pi)) + self.adv.reshape(-1, 1)
        acc = np.concatenate([np.angle(spec[..., :1]), phase[..., :-1]], -1).cumsum(-1)
        out = mag * np.exp(1j * acc)
        return np.stack([out.real, out.imag], -1).astype(np.float32)


class TimeStretch(AudioTensorOperation):
    def __init__(self, hop_length=None, n_freq=201, fixed_rate=None):
        self.n_freq = n_freq
        self.hop = hop_length if hop_length is not None else (n_freq - 1)
        self.rate = fixed_rate if fixed_rate is not None else 1.0
        if self.rate <= 0:
            raise ValueError("TimeStretch: fixed_rate must be positive")

    def _run(self, x):
        adv = np.linspace(0, math.pi * self.hop, self.n_freq)
        return PhaseVocoder(self.rate, adv)._run(x)


class Resample(AudioTensorOperation):
    """Band-limited (windowed-sinc) resampling from ``orig_freq`` to ``new_freq``."""

    def __init__(self, orig_freq=16000, new_freq=16000, resample_method=ResampleMethod.SINC_INTERPOLATION,
                 lowpass_filter_width=6, rolloff=0.99, beta=None):
        if orig_freq <= 0 or new_freq <= 0:
            raise ValueError("Resample: frequencies must be positive")
        self.orig, self.new = int(orig_freq), int(new_freq)
        self.method, self.width, self.rolloff, self.beta = _val(resample_method), lowpass_filter_width, rolloff, beta

    def _run(self, x):
        if self.orig == self.new:
            return x.astype(np.float32)
        g = math.gcd(self.orig, self.new)
        orig, new = self.orig // g, self.new // g
        base = min(orig, new) * self.rolloff
        width = int(math.ceil(self.width * orig / base))
        idx = np.arange(-width, width + orig, dtype=np.float64) / orig
        t = (np.arange(0, -new, -1, dtype=np.float64) / new)[:, None] + idx[None, :]
        t = np.clip(t * base, -self.width, self.width)
        if self.method == "kaiser_window":
            beta = 14.769656459379492 if self.beta is None else self.beta
            win = np.i0(beta * np.sqrt(np.maximum(1 - (t / self.width) ** 2, 0))) / np.i0(beta)
        else:
            win = np.cos(t * math.pi / self.width / 2) ** 2
        t = t * math.pi
        kernel = np.where(t == 0, 1.0, np.sin(t) / np.where(t == 0, 1.0, t)) * win * (base / orig)
        wav = _t(x).double()
        lead, n = wav.shape[:-1], wav.shape[-1]
        wav = torch.nn.functional.pad(wav.reshape(-1, 1, n), (width, width + orig))
        out = torch.nn.functional.conv1d(wav, torch.as_tensor(kernel)[:, None, :], stride=orig)
        out = out.transpose(1, 2).reshape(out.shape[0], -1)[:, :int(math.ceil(new * n / orig))]
        return out.reshape(lead + out.shape[-1:]).float().numpy()


class PitchShift(AudioTensorOperation):
    """Shifts pitch by ``n_steps`` (of ``bins_per_octave`` per octave): time-stretch by the inverse ratio with the
    phase vocoder, then resample back to the original length."""

    def __init__(self, sample_rate, n_steps, bins_per_octave=12, n_fft=512, win_length=None, hop_length=None,
                 window=WindowType.HANN):
        self.sr, self.rate = sample_rate, 2.0 ** (-float(n_steps) / bins_per_octave)
        self.n_fft, self.win = n_fft, win_length or n_fft
        self.hop, self.window = hop_length or (win_length or n_fft) // 4, window

    def _run(self, x):
        n = x.shape[-1]
        spec = Spectrogram(self.n_fft, self.win, self.hop, 0, self.window, None)._run(x)
        adv = np.linspace(0, math.pi * self.hop, self.n_fft // 2 + 1)
        stretched = PhaseVocoder(self.rate, adv)._run(spec)
        wav = InverseSpectrogram(None, self.n_fft, self.win, self.hop, 0, self.window)._run(stretched)
        out = Resample(int(round(self.sr / self.rate)), self.sr)._run(wav)
        if out.shape[-1] >= n:
            return out[..., :n]
        return np.pad(out, [(0, 0)] * (out.ndim - 1) + [(0, n - out.shape[-1])])


class _Unavailable(AudioTensorOperation):
    def __init__(self, *a, **k):
        raise NotImplementedError("%s is not provided (it reproduces a sox effect with internal state machines); the "
                                  "other transforms of this module cover filtering, spectral features and "
                                  "augmentation" % type(self).__name__)


class DetectPitchFrequency(AudioTensorOperation):
    """Pitch per frame from the normalised cross-correlation peak within [freq_low, freq_high], median-smoothed."""

    def __init__(self, sample_rate, frame_time=0.01, win_length=30, freq_low=85, freq_high=3400):
        self.sr, self.frame_time, self.win, self.lo, self.hi = sample_rate, frame_time, win_length, freq_low, freq_high

    def _run(self, x):
        lags = int(math.ceil(self.sr / self.lo))
        frame = int(math.ceil(self.sr * self.frame_time))
        n = x.shape[-1]
        count = int(math.ceil(n / frame))
        p = np.pad(x.astype(np.float64), [(0, 0)] * (x.ndim - 1) + [(0, lags + count * frame - n)])
        out = np.zeros(x.shape[:-1] + (count,), dtype=np.float32)
        min_lag = max(int(self.sr / self.hi), 1)
        for f in range(count):
            s0 = p[..., f * frame:f * frame + frame]
            best, best_lag = np.full(x.shape[:-1], -np.inf), np.ones(x.shape[:-1])
            for lag in range(min_lag, lags + 1):
                s1 = p[..., f * frame + lag:f * frame + lag + frame]
                if s1.shape[-1] < frame:
                    break
                corr = 2 * (s0 * s1).sum(-1) / (1e-9 + (s0 * s0).sum(-1) + (s1 * s1).sum(-1))
                better = corr > best + 0.01 * (lag > min_lag)
                best = np.where(better, corr, best)
                best_lag = np.where(better, lag, best_lag)
            out[..., f] = self.sr / best_lag
        half = self.win // 2
        padded = np.pad(out, [(0, 0)] * (out.ndim - 1) + [(half, half)], mode="edge")
        return np.stack([np.median(padded[..., i:i + self.win], -1) for i in range(count)], -1).astype(np.float32)


class Flanger(_Unavailable):
    pass


class Phaser(_Unavailable):
    pass


class Vad(_Unavailable):
    pass


__all__ = [n for n, v in list(globals().items()) if isinstance(v, type) and (issubclass(v, AudioTensorOperation)
                                                                             or issubclass(v, enum.Enum))
           and not n.startswith("_")] + ["melscale_fbanks", "linear_fbanks", "create_dct"]
