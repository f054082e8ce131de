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
