"""Turning prompts into atom byte strings. Reference: phyai/src/phyai/cache/radix_cache/encoding.py:15-128."""

from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Iterable, Sequence

_M64 = (1 << 64) - 1


@dataclass(frozen=True)
class ImageSegment:
    """``length`` placeholder positions starting at ``insert_position`` stand for one image whose content hash is (lo, hi)."""

    image_hash_lo: int
    image_hash_hi: int
    insert_position: int
    length: int


def page_align(atoms: bytes, page_bytes: int) -> tuple[bytes, int]:
    """Largest whole-page prefix and the number of bytes cut off."""
    if page_bytes <= 0:
        raise ValueError("page_bytes must be positive")
    keep = len(atoms) // page_bytes * page_bytes
    return atoms[:keep], len(atoms) - keep


def encode_text_atoms_int32(token_ids: Sequence[int]) -> bytes:
    return struct.pack(f"<{len(token_ids)}i", *(int(t) for t in token_ids))


def encode_eagle_bigram_atoms(token_ids: Sequence[int]) -> bytes:
    """N tokens -> N-1 atoms (token, next token): the key of a draft model's state."""
    ids = [int(t) for t in token_ids]
    return b"".join(struct.pack("<ii", a, b) for a, b in zip(ids, ids[1:]))


def encode_chunk_hash_atoms_u64(hashes: Iterable[int]) -> bytes:
    hs = [int(h) & _M64 for h in hashes]
    return struct.pack(f"<{len(hs)}Q", *hs)


def encode_image_hash_atom_sha256(digest: bytes) -> bytes:
    if len(digest) != 32:
        raise ValueError("digest must be 32 bytes")
    return bytes(digest)


def encode_prompt_to_atoms(text_token_ids: Sequence[int], image_segments: Sequence[ImageSegment]) -> bytes:
    """Mixed prompt -> 16-byte atoms (lo, hi): text = (token, 0); image position k = (hash_lo, hash_hi ^ k).
    Text and image atoms cannot collide while ``hash_hi`` is non-zero."""
    total = len(text_token_ids) + sum(s.length for s in image_segments)
    slots: list[tuple[int, int] | None] = [None] * total
    for seg in image_segments:
        if seg.insert_position < 0 or seg.insert_position + seg.length > total:
            raise ValueError(f"ImageSegment(at={seg.insert_position}, len={seg.length}) outside a prompt of {total}")
        for k in range(seg.length):
            slots[seg.insert_position + k] = (int(seg.image_hash_lo) & _M64, (int(seg.image_hash_hi) ^ k) & _M64)
    it = iter(text_token_ids)
    out = bytearray()
    for s in slots:
        if s is None:
            try:
                s = (int(next(it)) & _M64, 0)
            except StopIteration as e:
                raise ValueError("not enough text tokens for the non-image positions") from e
        out += struct.pack("<QQ", *s)
    return bytes(out)
