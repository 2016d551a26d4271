"""Audio front end: PCM decoding of WAV files, resampling to 16 kHz, and the log-mel spectrogram that speech
encoders consume.

The log-mel recipe is Whisper's: 25 ms Hann window (400 samples), 10 ms hop (160), power spectrum, 80 (or 128)
triangular mel filters on the Slaney scale with area normalisation, log10 clamped at 1e-10, dynamic range limited to
8 below the maximum, then ``(x + 4) / 4``.  The reference's audio stack decodes containers and builds the same
features on the CPU (zig/lib/audio/, zig/pkg/inference/src/pipelines/audio.zig:60-300); here the STFT and the
filterbank product are tensor ops on whatever device the waveform lives on (cuFFT + one small GEMM on the GPU).
"""
from __future__ import annotations

import io
import math
import struct
import wave
from typing import Tuple, Union

import torch

SAMPLE_RATE = 16000


def read_wav(data: Union[bytes, str]) -> Tuple[torch.Tensor, int]:
    """PCM WAV (8 / 16 / 24 / 32-bit integer, or 32-bit float) -> (mono float32 waveform in [-1, 1], sample rate)."""
    raw = open(data, "rb").read() if isinstance(data, str) else bytes(data)
    if len(raw) < 12 or raw[:4] != b"RIFF" or raw[8:12] != b"WAVE":
        raise ValueError("not a RIFF / WAVE file")
    fmt_tag = None
    pos = 12
    while pos + 8 <= len(raw):
        cid, size = raw[pos:pos + 4], struct.unpack("<I", raw[pos + 4:pos + 8])[0]
        if cid == b"fmt ":
            fmt_tag = struct.unpack("<H", raw[pos + 8:pos + 10])[0]
            if fmt_tag == 0xFFFE and size >= 26:                  # extensible: the real tag is in the sub-format
                fmt_tag = struct.unpack("<H", raw[pos + 32:pos + 34])[0]
            break
        pos += 8 + size + (size & 1)
    if fmt_tag == 3:                                              # IEEE float: the wave module refuses it
        ch, rate, bits = struct.unpack("<HI", raw[pos + 10:pos + 16]) + (struct.unpack("<H", raw[pos + 22:pos + 24])[0],)
        p = pos + 8 + struct.unpack("<I", raw[pos + 4:pos + 8])[0]
        while p + 8 <= len(raw) and raw[p:p + 4] != b"data":
            sz = struct.unpack("<I", raw[p + 4:p + 8])[0]
            p += 8 + sz + (sz & 1)
        n = struct.unpack("<I", raw[p + 4:p + 8])[0]
        if bits != 32:
            raise ValueError("only 32-bit float WAV is supported")
        x = torch.frombuffer(bytearray(raw[p + 8:p + 8 + n - n % 4]), dtype=torch.float32).clone()
    else:
        with wave.open(io.BytesIO(raw)) as w:
            ch, rate, width, n = w.getnchannels(), w.getframerate(), w.getsampwidth(), w.getnframes()
            buf = bytearray(w.readframes(n))
        if width == 1:
            x = (torch.frombuffer(buf, dtype=torch.uint8).float() - 128.0) / 128.0
        elif width == 2:
            x = torch.frombuffer(buf, dtype=torch.int16).float() / 32768.0
        elif width == 3:
            b = torch.frombuffer(buf, dtype=torch.uint8).view(-1, 3).int()
            v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
            x = torch.where(v >= 1 << 23, v - (1 << 24), v).float() / float(1 << 23)
        elif width == 4:
            x = torch.frombuffer(buf, dtype=torch.int32).float() / float(1 << 31)
        else:
            raise ValueError(f"unsupported sample width {width}")
    if ch > 1:
        x = x[: x.numel() // ch * ch].view(-1, ch).mean(1)
    return x.contiguous(), int(rate)


def resample(x: torch.Tensor, rate: int, target: int = SAMPLE_RATE, taps: int = 32) -> torch.Tensor:
    """Band-limited (Hann-windowed sinc) resampling: every output sample is a weighted sum of the ``2 * width + 1``
    input samples around its position, with the cut-off at the lower of the two Nyquist frequencies."""
    if rate == target:
        return x
    n_out = int(math.floor(x.numel() * target / rate))
    if n_out <= 0:
        return x.new_zeros(0)
    ratio = min(1.0, target / rate)                      # cut-off relative to the input Nyquist frequency
    width = int(math.ceil(taps / ratio))
    out = torch.empty(n_out, dtype=torch.float32, device=x.device)
    xp = torch.nn.functional.pad(x.float(), (width, width + 1))
    offs = torch.arange(-width, width + 1, device=x.device)
    for lo in range(0, n_out, 1 << 16):                  # blocks bound the [outputs, taps] gather
        n = torch.arange(lo, min(lo + (1 << 16), n_out), device=x.device, dtype=torch.float64)
        pos = n * (rate / target)
        base = pos.floor().long()
        u = (base[:, None] + offs[None, :]).double() - pos[:, None]          # input index - output position
        h = ratio * torch.sinc(ratio * u) * (0.5 + 0.5 * torch.cos(math.pi * u / (width + 1))).clamp(min=0.0)
        out[lo:lo + n.numel()] = (xp[base[:, None] + offs[None, :] + width] * h.float()).sum(1)
    return out


def _hz_to_mel(f: torch.Tensor) -> torch.Tensor:
    lin = f / (200.0 / 3)
    log = 15.0 + torch.log(f.clamp(min=1e-10) / 1000.0) / (math.log(6.4) / 27.0)
    return torch.where(f >= 1000.0, log, lin)


def _mel_to_hz(m: torch.Tensor) -> torch.Tensor:
    lin = m * (200.0 / 3)
    log = 1000.0 * torch.exp((m - 15.0) * (math.log(6.4) / 27.0))
    return torch.where(m >= 15.0, log, lin)


def mel_filterbank(n_mels: int = 80, n_fft: int = 400, rate: int = SAMPLE_RATE) -> torch.Tensor:
    """[n_fft / 2 + 1, n_mels] triangular filters, Slaney mel scale, each normalised by its bandwidth."""
    freqs = torch.linspace(0, rate / 2, n_fft // 2 + 1, dtype=torch.float64)
    mmin, mmax = _hz_to_mel(torch.tensor(0.0, dtype=torch.float64)), _hz_to_mel(torch.tensor(rate / 2, dtype=torch.float64))
    edges = _mel_to_hz(torch.linspace(float(mmin), float(mmax), n_mels + 2, dtype=torch.float64))
    diff = edges[1:] - edges[:-1]
    slopes = edges[None, :] - freqs[:, None]
    down = -slopes[:, :-2] / diff[:-1]
    up = slopes[:, 2:] / diff[1:]
    fb = torch.clamp(torch.minimum(down, up), min=0.0)
    fb = fb * (2.0 / (edges[2:] - edges[:-2]))[None, :]
    return fb.float()


_FB = {}


def log_mel(wave_16k: torch.Tensor, n_mels: int = 80, n_fft: int = 400, hop: int = 160,
            n_samples: int = 30 * SAMPLE_RATE) -> torch.Tensor:
    """Mono 16 kHz waveform -> [n_mels, n_samples / hop] log-mel features (zero-padded / cut to n_samples)."""
    x = wave_16k.float()
    if x.numel() < n_samples:
        x = torch.nn.functional.pad(x, (0, n_samples - x.numel()))
    x = x[:n_samples]
    key = (n_mels, n_fft, str(x.device))
    if key not in _FB:
        _FB[key] = (mel_filterbank(n_mels, n_fft).to(x.device), torch.hann_window(n_fft, device=x.device))
    fb, win = _FB[key]
    spec = torch.stft(x, n_fft, hop, window=win, center=True, pad_mode="reflect", return_complex=True)
    power = spec[:, :-1].abs().pow(2)                       # the last frame is dropped, as in the original recipe
    mel = fb.T @ power
    lg = torch.log10(mel.clamp(min=1e-10))
    lg = torch.maximum(lg, lg.max() - 8.0)
    return (lg + 4.0) / 4.0


# ---------------------------------------------------------------------------------------------------------
# CLAP front end: 48 kHz, 1024-point FFT, hop 480, 64 HTK mel bands over 50 Hz .. 14 kHz, power in dB.
CLAP_RATE, CLAP_FFT, CLAP_HOP, CLAP_MELS, CLAP_SECONDS = 48000, 1024, 480, 64, 10


def mel_filterbank_htk(n_mels: int, n_fft: int, rate: int, fmin: float, fmax: float) -> torch.Tensor:
    """[n_fft / 2 + 1, n_mels] triangular filters on the HTK mel scale (2595 log10(1 + f / 700)), not normalised."""
    to_mel = lambda f: 2595.0 * math.log10(1.0 + f / 700.0)
    freqs = torch.linspace(0, rate // 2, n_fft // 2 + 1, dtype=torch.float64)
    mels = torch.linspace(to_mel(fmin), to_mel(fmax), n_mels + 2, dtype=torch.float64)
    edges = 700.0 * (torch.pow(10.0, mels / 2595.0) - 1.0)
    diff = edges[1:] - edges[:-1]
    slopes = edges[None, :] - freqs[:, None]
    fb = torch.clamp(torch.minimum(-slopes[:, :-2] / diff[:-1], slopes[:, 2:] / diff[1:]), min=0.0)
    return fb.float()


def clap_log_mel(wave: torch.Tensor) -> torch.Tensor:
    """Mono 48 kHz waveform -> [frames, 64] mel power in dB (``10 log10(max(p, 1e-10))``), one frame per hop plus
    one (centred frames over a reflect-padded signal)."""
    x = wave.double()
    key = ("clap", str(x.device))
    if key not in _FB:
        _FB[key] = (mel_filterbank_htk(CLAP_MELS, CLAP_FFT, CLAP_RATE, 50.0, 14000.0).double().to(x.device),
                    torch.hann_window(CLAP_FFT, periodic=True, dtype=torch.float64, device=x.device))
    fb, win = _FB[key]
    spec = torch.stft(x, CLAP_FFT, CLAP_HOP, window=win, center=True, pad_mode="reflect", return_complex=True)
    mel = (spec.abs().pow(2).T @ fb).clamp(min=1e-10)
    return (10.0 * torch.log10(mel)).float()


def clap_features(wave_48k: torch.Tensor, channels: int = 4) -> Tuple[torch.Tensor, bool]:
    """Waveform -> ([channels, 1001, 64] features, is_longer), the input of the CLAP audio tower.

    Clips of at most ten seconds are repeated a whole number of times, zero-padded to ten seconds and their
    spectrogram is copied into every channel.  Longer clips are described by four planes: the whole spectrogram
    shrunk to 1001 frames (bilinear, half-pixel centres) and three ten-second crops taken at the front, the middle and
    the back -- fixed positions, where the training-time recipe drew them at random, so that an embedding is a
    function of the audio alone (zig/pkg/inference/src/pipelines/audio.zig:111 ``clapInputFeatures``, :270)."""
    n_max = CLAP_SECONDS * CLAP_RATE
    frames = n_max // CLAP_HOP + 1
    x = wave_48k.float().flatten()
    if x.numel() > n_max:
        mel = clap_log_mel(x)
        total = mel.shape[0]
        if total == frames:
            return mel[None].expand(max(channels, 4), -1, -1).contiguous(), False
        shrink = torch.nn.functional.interpolate(mel[None, None], size=(frames, CLAP_MELS), mode="bilinear",
                                                 align_corners=False)[0, 0]
        starts = [0, (total - frames) // 2, total - frames]
        planes = [shrink] + [mel[s:s + frames] for s in starts]
        out = torch.stack([planes[c % 4] for c in range(max(channels, 4))])
        return out, True
    if x.numel() == 0:
        x = torch.zeros(n_max)
    else:
        x = x.repeat(n_max // x.numel())
        x = torch.nn.functional.pad(x, (0, n_max - x.numel()))
    mel = clap_log_mel(x)
    return mel[None].expand(channels, -1, -1).contiguous(), False
