"""The FLAC writer of the speech endpoint, checked by a small decoder for the subset it emits (fixed
predictors, one Rice partition): sync codes, header CRC-8, frame CRC-16, STREAMINFO fields, the MD5
of the samples, and a bit-exact round trip of the 16-bit samples."""
import hashlib
import struct

import numpy as np
import torch

from vllm_omni_b200.entrypoints.openai.media_utils import _CRC8, _CRC16, _utf8_number, encode_audio, flac_bytes


class Bits:
    def __init__(self, data):
        self.b = np.unpackbits(np.frombuffer(data, dtype=np.uint8))
        self.p = 0

    def u(self, n):
        v = 0
        for bit in self.b[self.p:self.p + n]:
            v = (v << 1) | int(bit)
        self.p += n
        return v

    def s(self, n):
        v = self.u(n)
        return v - (1 << n) if v >> (n - 1) else v

    def unary(self):
        q = 0
        while self.b[self.p] == 0:
            q += 1
            self.p += 1
        self.p += 1
        return q


def decode(data):
    assert data[:4] == b"fLaC" and data[4] == 0x80 and int.from_bytes(data[5:8], "big") == 34
    r = Bits(data[8:42])
    info = dict(min_block=r.u(16), max_block=r.u(16), min_frame=r.u(24), max_frame=r.u(24), rate=r.u(20), ch=r.u(3) + 1,
                bps=r.u(5) + 1, total=r.u(36), md5=data[26:42])
    pos, chans, frame_no = 42, [[] for _ in range(info["ch"])], 0
    while pos < len(data):
        r = Bits(data[pos:])
        assert r.u(15) == 0x7FFC and r.u(1) == 0
        bs_code, sr_code = r.u(4), r.u(4)
        ch, ss, _ = r.u(4) + 1, r.u(3), r.u(1)
        assert bs_code == 7 and ss == 4 and ch == info["ch"]
        first = r.u(8)
        n_extra = 0 if first < 0x80 else (8 - len(bin(first ^ 0xFF)) + 2) - 1
        num = first if first < 0x80 else first & (0x7F >> (n_extra + 1))
        for _ in range(n_extra):
            num = (num << 6) | (r.u(8) & 0x3F)
        assert num == frame_no
        n = r.u(16) + 1
        hdr_len = r.p // 8
        crc = 0
        for b in data[pos:pos + hdr_len]:
            crc = _CRC8[crc ^ b]
        assert crc == r.u(8)
        for c in range(ch):
            assert r.u(1) == 0
            typ = r.u(6)
            assert r.u(1) == 0 and 8 <= typ <= 12
            order = typ - 8
            out = [r.s(16) for _ in range(order)]
            assert r.u(2) == 0 and r.u(4) == 0
            k = r.u(4)
            for _ in range(n - order):
                u = (r.unary() << k) | (r.u(k) if k else 0)
                res = (u >> 1) if not u & 1 else -((u + 1) >> 1)
                pred = 0 if order == 0 else (out[-1] if order == 1 else 2 * out[-1] - out[-2])
                out.append(pred + res)
            chans[c] += out
        r.p = (r.p + 7) // 8 * 8
        end = pos + r.p // 8
        crc = 0
        for b in data[pos:end]:
            crc = ((crc << 8) & 0xFFFF) ^ _CRC16[(crc >> 8) ^ b]
        assert crc == struct.unpack(">H", data[end:end + 2])[0]
        assert info["min_frame"] <= end + 2 - pos <= info["max_frame"]
        pos, frame_no = end + 2, frame_no + 1
    return info, np.array(chans)


def test_flac_round_trip_mono_and_stereo():
    t = torch.arange(10000) / 24000
    mono = 0.4 * torch.sin(2 * torch.pi * 220 * t) + 0.01 * torch.randn(10000)
    data = flac_bytes(mono, 24000)
    info, pcm = decode(data)
    want = (np.clip(mono.numpy(), -1, 1) * 32767.0).astype(np.int64)
    assert info["rate"] == 24000 and info["ch"] == 1 and info["bps"] == 16 and info["total"] == 10000
    assert np.array_equal(pcm[0], want) and info["md5"] == hashlib.md5(want.astype("<i2").tobytes()).digest()
    assert len(data) < 0.8 * 2 * 10000                       # smaller than the raw 16-bit samples
    stereo = torch.stack([mono, -0.5 * mono.roll(7)])
    info, pcm = decode(flac_bytes(stereo, 44100, block=1024))
    want = (np.clip(stereo.numpy(), -1, 1) * 32767.0).astype(np.int64)
    assert info["ch"] == 2 and info["rate"] == 44100 and np.array_equal(pcm, want)
    assert info["md5"] == hashlib.md5(want.T.astype("<i2").tobytes()).digest()
    data, media = encode_audio(mono, 24000, "flac")
    assert media == "audio/flac" and data[:4] == b"fLaC"


def test_frame_numbers_beyond_one_byte_and_silence():
    assert _utf8_number(0x7F) == [0x7F] and _utf8_number(0x80) == [0xC2, 0x80] and _utf8_number(0x800) == [0xE0, 0xA0, 0x80]
    x = torch.zeros(300 * 16)
    x[1000:1100] = 0.25
    info, pcm = decode(flac_bytes(x, 16000, block=16))       # 300 frames: numbers need two bytes from 128 on
    assert info["total"] == 4800 and np.array_equal(pcm[0], (x.numpy() * 32767.0).astype(np.int64))
