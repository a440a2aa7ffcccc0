"""PNG writer (8-bit RGB / RGBA / gray, tEXt chunks for generation parameters) and a decoder for the same subset,
plus a WAV (PCM16 / float32) writer. No imaging library is needed.

The writer takes the role of serenitymojo/image/png.mojo (CRC/Adler framed PNG with tEXt ``serenity.genparams.v1``
metadata as used by the serving backends, serenity-server/README.md:23-37), the decoder of
serenitymojo/image/decode.mojo, the WAV writer of serenitymojo/audio/wav.mojo.
"""
from __future__ import annotations

import struct
import zlib
from typing import Dict, Optional, Tuple

import numpy as np
import torch

_SIG = b"\x89PNG\r\n\x1a\n"


def _chunk(tag: bytes, data: bytes) -> bytes:
    return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)


def encode_png(img, text: Optional[Dict[str, str]] = None, compress_level: int = 6) -> bytes:
    """img: uint8 array / tensor [H, W], [H, W, 3] or [H, W, 4]."""
    a = img.detach().cpu().numpy() if isinstance(img, torch.Tensor) else np.asarray(img)
    if a.dtype != np.uint8:
        raise ValueError("encode_png wants uint8")
    if a.ndim == 2:
        a = a[:, :, None]
    h, w, c = a.shape
    ctype = {1: 0, 3: 2, 4: 6}[c]
    raw = np.concatenate([np.zeros((h, 1), np.uint8), a.reshape(h, w * c)], axis=1).tobytes()  # filter 0 per row
    out = [_SIG, _chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, ctype, 0, 0, 0))]
    for k, v in (text or {}).items():
        out.append(_chunk(b"tEXt", k.encode("latin-1") + b"\x00" + v.encode("latin-1", "replace")))
    out.append(_chunk(b"IDAT", zlib.compress(raw, compress_level)))
    out.append(_chunk(b"IEND", b""))
    return b"".join(out)


def save_png(path, img, text: Optional[Dict[str, str]] = None) -> None:
    with open(path, "wb") as f:
        f.write(encode_png(img, text))


def tensor_to_uint8(x: torch.Tensor) -> torch.Tensor:
    """[C, H, W] or [H, W, C] float in [-1, 1] -> uint8 [H, W, C]."""
    if x.dim() == 3 and x.shape[0] in (1, 3, 4) and x.shape[-1] not in (1, 3, 4):
        x = x.permute(1, 2, 0)
    return ((x.float().clamp(-1, 1) + 1.0) * 127.5).round().to(torch.uint8).cpu()


def _paeth(a, b, c):
    p = a + b - c
    pa, pb, pc = abs(p - a), abs(p - b), abs(p - c)
    return a if (pa <= pb and pa <= pc) else (b if pb <= pc else c)


def decode_png(data: bytes) -> Tuple[np.ndarray, Dict[str, str]]:
    """Returns (uint8 [H, W, C], tEXt dict). 8-bit gray / RGB / RGBA, non-interlaced."""
    if data[:8] != _SIG:
        raise ValueError("not a PNG")
    pos, idat, text, hdr = 8, [], {}, None
    while pos < len(data):
        (n,) = struct.unpack_from(">I", data, pos)
        tag = data[pos + 4:pos + 8]
        body = data[pos + 8:pos + 8 + n]
        (crc,) = struct.unpack_from(">I", data, pos + 8 + n)
        if zlib.crc32(tag + body) & 0xFFFFFFFF != crc:
            raise ValueError(f"bad CRC in {tag!r}")
        if tag == b"IHDR":
            hdr = struct.unpack(">IIBBBBB", body)
        elif tag == b"IDAT":
            idat.append(body)
        elif tag == b"tEXt":
            k, _, v = body.partition(b"\x00")
            text[k.decode("latin-1")] = v.decode("latin-1")
        elif tag == b"IEND":
            break
        pos += 12 + n
    w, h, depth, ctype, _, _, interlace = hdr
    if depth != 8 or interlace != 0 or ctype not in (0, 2, 6):
        raise ValueError("unsupported PNG variant")
    c = {0: 1, 2: 3, 6: 4}[ctype]
    raw = zlib.decompress(b"".join(idat))
    stride = w * c
    out = np.zeros((h, stride), np.uint8)
    prev = np.zeros(stride, np.int32)
    for y in range(h):
        f = raw[y * (stride + 1)]
        line = np.frombuffer(raw, np.uint8, stride, y * (stride + 1) + 1).astype(np.int32)
        if f == 0:
            cur = line
        elif f == 2:
            cur = (line + prev) & 255
        else:
            cur = np.zeros(stride, np.int32)
            for i in range(stride):
                a = cur[i - c] if i >= c else 0
                b = prev[i]
                cc = prev[i - c] if i >= c else 0
                if f == 1:
                    pred = a
                elif f == 3:
                    pred = (a + b) // 2
                else:
                    pred = _paeth(int(a), int(b), int(cc))
                cur[i] = (line[i] + pred) & 255
        out[y] = cur.astype(np.uint8)
        prev = cur
    return out.reshape(h, w, c), text


def load_png(path) -> Tuple[np.ndarray, Dict[str, str]]:
    with open(path, "rb") as f:
        return decode_png(f.read())


def save_wav(path, samples, sample_rate: int = 44100, float32: bool = False) -> None:
    """samples: [T] or [T, channels] float in [-1, 1]."""
    a = samples.detach().cpu().numpy() if isinstance(samples, torch.Tensor) else np.asarray(samples)
    if a.ndim == 1:
        a = a[:, None]
    ch = a.shape[1]
    if float32:
        body, fmt, bits = a.astype("<f4").tobytes(), 3, 32
    else:
        body, fmt, bits = (np.clip(a, -1, 1) * 32767.0).round().astype("<i2").tobytes(), 1, 16
    byte_rate = sample_rate * ch * bits // 8
    hdr = b"RIFF" + struct.pack("<I", 36 + len(body)) + b"WAVE" + b"fmt " + struct.pack(
        "<IHHIIHH", 16, fmt, ch, sample_rate, byte_rate, ch * bits // 8, bits) + b"data" + struct.pack("<I", len(body))
    with open(path, "wb") as f:
        f.write(hdr + body)
