"""Host model of a GPU replica, built on the host codec: what the round kernel has to reproduce bit for bit.
Used by the kernel tests (against the device) and by the protocol tests (replicas of this model talking to each other)."""
import torch


class Oracle:
    """Host model of a replica: values, one mirror per link, frames exchanged as (codes or words, scales), and the
    change mark of every 4096-element tile.  A link is told about a tile only while the tile carries a mark: set by
    whatever changes the values or a mirror from outside the rounds, kept while a visit still found something to say;
    a frame that merely arrives (it moves values and mirror alike) does not make the tile speak."""

    def __init__(self, core, n, block, n_links, bits=8, min_exp=-60, rel_bits=22):
        self.core, self.n, self.block, self.bits = core, n, block, bits
        self.v = torch.zeros(n)
        self.k = [torch.zeros(n) for _ in range(n_links)]
        self.min_exp, self.rel_bits = min_exp, rel_bits
        self.dirty = torch.ones((n + 4095) // 4096, dtype=torch.bool)  # a fresh replica, a new edge: everything is looked at

    def mark(self):
        self.dirty[:] = True

    def encode(self, link):
        k_before = self.k[link].clone()
        codes, scales = self._encode_all(link)
        spt = 4096 // self.block
        for t in range(self.dirty.numel()):
            lo, hi = t * 4096, min((t + 1) * 4096, self.n)
            if not bool(self.dirty[t]):
                self.k[link][lo:hi] = k_before[lo:hi]
                scales[t * spt:(t + 1) * spt] = 0
                if self.bits == 1:
                    codes[lo // 32:(hi + 31) // 32] = 0
                else:
                    codes[lo:hi] = 1 << (self.bits - 1)
            else:
                self.dirty[t] = bool(scales[t * spt:(t + 1) * spt].any())
        return codes, scales

    def _encode_all(self, link):
        scales = torch.zeros(self.core.block_scales(self.n, self.block), dtype=torch.uint8)
        if self.bits == 1:
            codes = torch.zeros(self.core.block_words(self.n), dtype=torch.int32)
            self.core.encode_block(self.v.data_ptr(), self.k[link].data_ptr(), self.n, self.block, self.min_exp, self.rel_bits,
                                   codes.data_ptr(), scales.data_ptr())
        else:
            codes = torch.zeros(self.n, dtype=torch.uint8)
            self.core.encode_block_int(self.v.data_ptr(), self.k[link].data_ptr(), self.n, self.block, self.min_exp, self.rel_bits,
                                       self.bits, codes.data_ptr(), scales.data_ptr())
        return codes, scales

    def steps(self, frame):
        codes, scales = frame
        out = torch.zeros(self.n)
        if self.bits == 1:
            self.core.block_sign_steps(codes.data_ptr(), scales.data_ptr(), self.n, self.block, out.data_ptr())
        else:
            self.core.block_int_steps(codes.data_ptr(), scales.data_ptr(), self.n, self.block, self.bits, out.data_ptr())
        return out

    def decode(self, link, frames):
        """What one sweep does with the frames it finds on a link: their steps are added up first (in order), the sum
        then goes into the values and into the link's mirror."""
        if not isinstance(frames, list):
            frames = [frames]
        if not frames:
            return
        acc = torch.zeros(self.n)
        for fr in frames:
            acc = acc + self.steps(fr)
        self.v += acc
        self.k[link] += acc

    def payload_of_tile(self, frame, tile):
        """(code words as the ring slot holds them, scale bytes, mask of 32-element chunks whose block is not silent)."""
        codes, scales = frame
        lo, hi = tile * 4096, min((tile + 1) * 4096, self.n)
        if self.bits == 1:
            unpacked = torch.zeros(4096, dtype=torch.uint8)
            w = codes[lo // 32:(hi + 31) // 32].to(torch.int64) & 0xFFFFFFFF
            bits = ((w[:, None] >> torch.arange(32)) & 1).reshape(-1).to(torch.uint8)
            unpacked[:bits.numel()] = bits
        else:
            unpacked = torch.full((4096,), 1 << (self.bits - 1), dtype=torch.uint8)
            unpacked[:hi - lo] = codes[lo:hi]
        words = torch.zeros(self.bits * 128, dtype=torch.int32)
        self.core.pack_tile_codes(unpacked.data_ptr(), self.bits, words.data_ptr())
        spt = 4096 // self.block
        sc = torch.zeros(spt, dtype=torch.uint8)
        mine = scales[tile * spt:(tile + 1) * spt]
        sc[:mine.numel()] = mine
        loud = (sc != 0).repeat_interleave(self.block // 32)
        return words, sc, loud

    # ------------------------------------------------------------------------------------------
    def tiles_of(self, frame):
        """Mask of the tiles a frame has anything for (a tile whose blocks are all silent is not sent at all)."""
        _, scales = frame
        spt = 4096 // self.block
        pad = torch.zeros(self.dirty.numel() * spt, dtype=torch.uint8)
        pad[:scales.numel()] = scales
        return pad.reshape(-1, spt).ne(0).any(1)

    def visit(self, arrived=None):
        """One pass over the tensor.  `arrived`: {link: [frames]} found in the in-rings.  Returns {link: frame} for the
        links that were told something (frames that say nothing anywhere are left out).  What arrived goes into the
        values and into the mirror of the link it came on; a link then hears about a tile if the tile carries a
        change mark or if something for it arrived on another link."""
        arrived = {l: fr for l, fr in sorted((arrived or {}).items()) if fr}
        came = {l: torch.zeros_like(self.dirty) for l in arrived}
        total = torch.zeros(self.n)   # everything that arrived, added up ring by ring and frame by frame, goes into
        for l, frames in arrived.items():  # the values as one sum; what arrived on a link goes into that link's mirror
            acc = torch.zeros(self.n)
            for fr in frames:
                came[l] |= self.tiles_of(fr)
                st = self.steps(fr)
                acc = acc + st
                total = total + st
            self.k[l] += acc
        self.v += total
        marks = self.dirty.clone()
        still = torch.zeros_like(self.dirty)
        out = {}
        spt = 4096 // self.block
        for l in range(len(self.k)):
            want = marks.clone()
            for j, m in came.items():
                if j != l:
                    want |= m
            self.dirty = want.clone()
            frame = self.encode(l)          # leaves in self.dirty the wanted tiles that still had something to say
            still |= self.dirty
            if bool(frame[1].any()):
                out[l] = frame
        self.dirty = still
        return out
