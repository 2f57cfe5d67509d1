"""Audio transforms against closed forms / numpy / scipy."""
import math

import numpy as np
import pytest
import scipy.signal

from mindspore_b200.dataset import audio


def _sine(freq, sr=8000, n=4000, amp=0.5):
    return (amp * np.sin(2 * math.pi * freq * np.arange(n) / sr)).astype(np.float32)[None]


def test_filters():
    sr = 8000
    low, high = _sine(100, sr), _sine(3000, sr)
    lp = audio.LowpassBiquad(sr, 500.0)
    assert np.abs(lp(low)[0, 1000:]).max() > 0.45 and np.abs(lp(high)[0, 1000:]).max() < 0.02
    hp = audio.HighpassBiquad(sr, 1500.0)
    assert np.abs(hp(low)[0, 1000:]).max() < 0.02 and np.abs(hp(high)[0, 1000:]).max() > 0.4
    notch = audio.BandrejectBiquad(sr, 1000.0, 0.5)
    assert np.abs(notch(_sine(1000, sr))[0, 2000:]).max() < 0.02
    eq = audio.EqualizerBiquad(sr, 1000.0, 6.0, 0.707)
    assert abs(np.abs(eq(_sine(1000, sr))[0, 2000:]).max() / 0.5 - 10 ** (6 / 20)) < 0.03
    x = np.random.RandomState(0).uniform(-0.1, 0.1, (2, 200)).astype(np.float32)
    got = audio.LFilter([1.0, -0.5], [0.3, 0.2])(x)
    np.testing.assert_allclose(got, scipy.signal.lfilter([0.3, 0.2], [1.0, -0.5], x), atol=1e-6)
    np.testing.assert_allclose(audio.Biquad(0.3, 0.2, 0.0, 1.0, -0.5, 0.0)(x), got, atol=1e-6)
    assert audio.Filtfilt([1.0, -0.5], [0.3, 0.2])(x).shape == x.shape
    riaa = audio.RiaaBiquad(44100)
    assert abs(np.abs(riaa(_sine(1000, 44100, 8000, 0.2))[0, 4000:]).max() / 0.2 - 1.0) < 0.02   # unit gain at 1 kHz
    with pytest.raises(ValueError):
        audio.LowpassBiquad(sr, 500.0, 0.0)
    with pytest.raises(ValueError):
        audio.DeemphBiquad(8000)
    assert audio.BandBiquad(sr, 1000.0)(low).shape == low.shape and audio.DeemphBiquad(44100)(low).shape == low.shape


def test_level_and_companding():
    x = np.array([[0.0, 0.25, -0.5, 1.0]], np.float32)
    np.testing.assert_allclose(audio.Gain(6.0)(x), x * 10 ** 0.3, rtol=1e-6)
    np.testing.assert_allclose(audio.Vol(0.5)(x), x * 0.5)
    np.testing.assert_allclose(audio.Vol(-6.0, audio.GainType.DB)(x), x * 10 ** -0.3, rtol=1e-6)
    np.testing.assert_allclose(audio.DCShift(0.25)(x), np.clip(x + 0.25, -1, 1))
    enc = audio.MuLawEncoding(256)(x)
    assert enc.dtype == np.int32 and enc.min() >= 0 and enc.max() <= 255
    np.testing.assert_allclose(audio.MuLawDecoding(256)(enc), x, atol=0.02)
    db = audio.AmplitudeToDB(top_db=None)(np.array([[[1.0, 10.0, 100.0]]], np.float32))
    np.testing.assert_allclose(db, [[[0, 10, 20]]], atol=1e-5)
    np.testing.assert_allclose(audio.DBToAmplitude(1.0, 1.0)(db), [[[1, 10, 100]]], rtol=1e-5)
    c = np.array([[3.0, 4.0]], np.float32)
    np.testing.assert_allclose(audio.ComplexNorm(2.0)(c), [25.0])
    mag, ph = audio.Magphase()(c)
    np.testing.assert_allclose(mag, [5.0]) and np.testing.assert_allclose(ph, [math.atan2(4, 3)], rtol=1e-6)
    faded = audio.Fade(2, 2)(np.ones((1, 6), np.float32))
    np.testing.assert_allclose(faded[0], [0, 1, 1, 1, 1, 0])
    d = audio.ComputeDeltas(3)(np.array([[0.0, 1.0, 2.0, 3.0]], np.float32))
    np.testing.assert_allclose(d[0, 1:3], [1, 1])
    assert np.abs(audio.Dither()(x) - x).max() <= 2.0 / 2 ** 15 + 1e-6
    assert audio.Contrast()(x).shape == x.shape and audio.Overdrive()(x).shape == x.shape


def test_spectral_features():
    sr = 8000
    x = _sine(1000, sr, 4000)
    spec = audio.Spectrogram(n_fft=256, hop_length=128)(x)
    assert spec.shape == (1, 129, 4000 // 128 + 1)
    assert int(spec[0, :, 10].argmax()) == round(1000 / (sr / 256))
    mel = audio.MelSpectrogram(sr, n_fft=256, hop_length=128, n_mels=20)(x)
    assert mel.shape == (1, 20, spec.shape[-1]) and mel.min() >= 0
    fb = audio.melscale_fbanks(129, 0.0, 4000.0, 20, sr)
    assert fb.shape == (129, 20) and fb.min() >= 0 and (fb.sum(0) > 0).all()
    dct = audio.create_dct(5, 20, audio.NormMode.ORTHO)
    np.testing.assert_allclose(dct.T @ dct, np.eye(5), atol=1e-5)
    assert audio.MFCC(sr, n_mfcc=13, melkwargs={"n_fft": 256, "hop_length": 128, "n_mels": 20})(x).shape[1] == 13
    assert audio.LFCC(sr, n_filter=20, n_lfcc=8, speckwargs={"n_fft": 256, "hop_length": 128})(x).shape[1] == 8
    cen = audio.SpectralCentroid(sr, n_fft=256, hop_length=128)(x)
    assert abs(float(cen[0, 10]) - 1000) < 40
    comp = audio.Spectrogram(n_fft=256, hop_length=64, power=None)(x)
    back = audio.InverseSpectrogram(4000, n_fft=256, hop_length=64)(comp)
    np.testing.assert_allclose(back, x, atol=1e-4)
    gl = audio.GriffinLim(n_fft=256, hop_length=64, n_iter=8, length=4000)(audio.Spectrogram(256, hop_length=64)(x))
    assert gl.shape == (1, 4000)
    inv = audio.InverseMelScale(129, 20, sr)(audio.MelScale(20, sr, n_stft=129)(spec))
    assert inv.shape == spec.shape and int(inv[0, :, 10].argmax()) in range(30, 35)
    stretched = audio.TimeStretch(hop_length=64, n_freq=129, fixed_rate=2.0)(comp)
    assert stretched.shape[-2] == math.ceil(comp.shape[-2] / 2)
    pitch = audio.DetectPitchFrequency(sr, freq_low=200, freq_high=2000)(_sine(400, sr, 2000))
    assert abs(float(np.median(pitch)) - 400) < 25


def test_resample_pitch_and_masks():
    sr = 8000
    x = _sine(500, sr, 4000)
    up = audio.Resample(sr, 16000)(x)
    assert up.shape == (1, 8000)
    ref = _sine(500, 16000, 8000)
    np.testing.assert_allclose(up[0, 200:-200], ref[0, 200:-200], atol=0.01)
    down = audio.Resample(sr, 4000, audio.ResampleMethod.KAISER_WINDOW)(x)
    assert down.shape == (1, 2000)
    shifted = audio.PitchShift(sr, 12, n_fft=256)(x)
    spec = audio.Spectrogram(n_fft=512, hop_length=256)(shifted)
    assert shifted.shape == x.shape and abs(int(spec[0, :, 5].argmax()) * sr / 512 - 1000) < 60
    s = np.ones((2, 10, 20), np.float32)
    t = audio.TimeMasking(False, 5, 3)(s)
    assert t[:, :, :3].min() == 1 and t.shape == s.shape and (t == 0).sum() % 20 == 0
    f = audio.FrequencyMasking(True, 4)(s)
    assert f.shape == s.shape
    m = audio.MaskAlongAxis(2, 3, 0.0, 2)(s)
    assert (m[:, :, 2:5] == 0).all() and m.sum() == s.sum() - 2 * 10 * 3
    assert audio.MaskAlongAxisIID(4, 0.0, 1)(s).shape == s.shape
    cmn = audio.SlidingWindowCmn(cmn_window=4, center=True)(np.arange(24, dtype=np.float32).reshape(1, 6, 4))
    assert cmn.shape == (1, 6, 4) and float(cmn[0, 3].sum()) == 8.0   # row 3 minus the mean of rows 1..4
    with pytest.raises(NotImplementedError):
        audio.Vad(8000)
