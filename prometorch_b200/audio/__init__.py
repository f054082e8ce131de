"""Audio helpers: STFT / inverse STFT, mel filterbank and MFCC, resampling, 16-bit PCM WAV I/O (torch/audio/*.h)."""
from __future__ import annotations

import math
import struct

import torch


def stft(x: torch.Tensor, n_fft: int = 400, hop_length: int = 160, window: torch.Tensor = None) -> torch.Tensor:
    window = torch.hann_window(n_fft, device=x.device) if window is None else window
    return torch.stft(x, n_fft, hop_length, window=window, return_complex=True)


def istft(spec: torch.Tensor, n_fft: int = 400, hop_length: int = 160, window: torch.Tensor = None, length: int = None) -> torch.Tensor:
    window = torch.hann_window(n_fft, device=spec.device) if window is None else window
    return torch.istft(spec, n_fft, hop_length, window=window, length=length)


def _hz_to_mel(f):
    return 2595.0 * math.log10(1.0 + f / 700.0)


def mel_filterbank(n_mels: int, n_fft: int, sample_rate: int) -> torch.Tensor:
    mels = torch.linspace(_hz_to_mel(0.0), _hz_to_mel(sample_rate / 2), n_mels + 2)
    hz = 700.0 * (10 ** (mels / 2595.0) - 1.0)
    bins = torch.floor((n_fft + 1) * hz / sample_rate).long()
    fb = torch.zeros(n_mels, n_fft // 2 + 1)
    for m in range(1, n_mels + 1):
        l, c, r = int(bins[m - 1]), int(bins[m]), int(bins[m + 1])
        for k in range(l, c):
            fb[m - 1, k] = (k - l) / max(c - l, 1)
        for k in range(c, r):
            fb[m - 1, k] = (r - k) / max(r - c, 1)
    return fb


def mfcc(x: torch.Tensor, sample_rate: int = 16000, n_mfcc: int = 13, n_mels: int = 40, n_fft: int = 400, hop_length: int = 160) -> torch.Tensor:
    power = stft(x, n_fft, hop_length).abs() ** 2
    mel = torch.matmul(mel_filterbank(n_mels, n_fft, sample_rate).to(x.device), power)
    logmel = torch.log(mel + 1e-10)
    n = torch.arange(n_mels, device=x.device)
    dct = torch.cos(math.pi / n_mels * (n[None, :] + 0.5) * torch.arange(n_mfcc, device=x.device)[:, None]) * math.sqrt(2.0 / n_mels)
    return torch.matmul(dct, logmel)


def resample(x: torch.Tensor, orig_rate: int, new_rate: int) -> torch.Tensor:
    n = int(round(x.shape[-1] * new_rate / orig_rate))
    return torch.nn.functional.interpolate(x.reshape(1, 1, -1), size=n, mode="linear", align_corners=False).reshape(*x.shape[:-1], n)


def save_wav(path: str, x: torch.Tensor, sample_rate: int = 16000):
    pcm = (x.clamp(-1, 1) * 32767).to(torch.int16).cpu().numpy().tobytes()
    with open(path, "wb") as f:
        f.write(b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, 1, sample_rate, sample_rate * 2, 2, 16))
        f.write(b"data" + struct.pack("<I", len(pcm)) + pcm)


def load_wav(path: str):
    with open(path, "rb") as f:
        b = f.read()
    sr = struct.unpack_from("<I", b, 24)[0]
    i = b.find(b"data")
    n = struct.unpack_from("<I", b, i + 4)[0]
    x = torch.frombuffer(bytearray(b[i + 8:i + 8 + n]), dtype=torch.int16).float() / 32767.0
    return x, sr


# ---------------------------------------------------------------------------------------------- functional (torch/audio/functional.h)
def hann_window(n: int, device=None) -> torch.Tensor:
    return torch.hann_window(n, device=device)


def spectrogram(x: torch.Tensor, n_fft: int = 400, hop_length: int = 160, window: torch.Tensor = None, power: float = 2.0) -> torch.Tensor:
    """|STFT|^power, ``[..., n_fft/2 + 1, frames]`` (power None: the complex STFT)."""
    s = stft(x, n_fft, hop_length, window)
    return s if power is None else s.abs() ** power


def melscale_fbanks(n_freqs: int, n_mels: int, sample_rate: int) -> torch.Tensor:
    """Triangular mel filters as ``[n_freqs, n_mels]`` (the orientation of the reference's function; ``mel_filterbank`` is its transpose)."""
    return mel_filterbank(n_mels, (n_freqs - 1) * 2, sample_rate).t().contiguous()


def amplitude_to_db(x: torch.Tensor, multiplier: float = 10.0, amin: float = 1e-10, db_multiplier: float = 0.0, top_db: float = None) -> torch.Tensor:
    db = multiplier * torch.log10(x.clamp_min(amin)) - multiplier * db_multiplier
    if top_db is not None:
        db = torch.maximum(db, db.amax() - top_db)
    return db


def mu_law_encoding(x: torch.Tensor, quantization_channels: int = 256) -> torch.Tensor:
    """Signal in [-1, 1] -> integers in [0, quantization_channels)."""
    mu = quantization_channels - 1.0
    y = torch.sign(x) * torch.log1p(mu * x.abs().clamp(max=1.0)) / math.log1p(mu)
    return ((y + 1) / 2 * mu + 0.5).to(torch.int64)


def mu_law_decoding(q: torch.Tensor, quantization_channels: int = 256) -> torch.Tensor:
    mu = quantization_channels - 1.0
    y = q.to(torch.float32) / mu * 2 - 1
    return torch.sign(y) * (torch.exp(y.abs() * math.log1p(mu)) - 1) / mu


# ---------------------------------------------------------------------------------------------- transforms (torch/audio/transforms.h)
class Spectrogram(torch.nn.Module):
    def __init__(self, n_fft: int = 400, hop_length: int = None, power: float = 2.0):
        super().__init__()
        self.n_fft, self.hop_length, self.power = n_fft, hop_length or n_fft // 2, power
        self.register_buffer("window", torch.hann_window(n_fft))

    def forward(self, x):
        return spectrogram(x, self.n_fft, self.hop_length, self.window, self.power)


class MelSpectrogram(torch.nn.Module):
    def __init__(self, sample_rate: int = 16000, n_fft: int = 400, hop_length: int = None, n_mels: int = 128):
        super().__init__()
        self.spec = Spectrogram(n_fft, hop_length, 2.0)
        self.register_buffer("fb", mel_filterbank(n_mels, n_fft, sample_rate))

    def forward(self, x):
        return torch.matmul(self.fb, self.spec(x))


class AmplitudeToDB(torch.nn.Module):
    def __init__(self, stype: str = "power", top_db: float = None):
        super().__init__()
        self.multiplier, self.top_db = (10.0 if stype == "power" else 20.0), top_db

    def forward(self, x):
        return amplitude_to_db(x, self.multiplier, top_db=self.top_db)


class MFCC(torch.nn.Module):
    def __init__(self, sample_rate: int = 16000, n_mfcc: int = 40, n_mels: int = 128, n_fft: int = 400, hop_length: int = None):
        super().__init__()
        self.mel, self.to_db = MelSpectrogram(sample_rate, n_fft, hop_length, n_mels), AmplitudeToDB("power", 80.0)
        n = torch.arange(n_mels)
        dct = torch.cos(math.pi / n_mels * (n[None, :] + 0.5) * torch.arange(n_mfcc)[:, None]) * math.sqrt(2.0 / n_mels)
        dct[0] *= 1.0 / math.sqrt(2.0)                                  # orthonormal DCT-II
        self.register_buffer("dct", dct)

    def forward(self, x):
        return torch.matmul(self.dct, self.to_db(self.mel(x)))


class Resample(torch.nn.Module):
    def __init__(self, orig_freq: int = 16000, new_freq: int = 16000):
        super().__init__()
        self.orig_freq, self.new_freq = orig_freq, new_freq

    def forward(self, x):
        return x if self.orig_freq == self.new_freq else resample(x, self.orig_freq, self.new_freq)
