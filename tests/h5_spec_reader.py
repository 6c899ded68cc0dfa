"""Independent, minimal HDF5 reader written only for the tests: a second implementation of the parts of the file
format that the C++ store emits (superblock v0, v1 object headers, old-style groups, chunked + deflate datasets,
scalar attributes with variable-length strings). It shares no code with csrc/h5/h5store.cc."""
import struct
import zlib

import numpy as np

UNDEF = 0xFFFFFFFFFFFFFFFF


class SpecReader:
    def __init__(self, path):
        self.b = open(path, "rb").read()
        assert self.b[:8] == b"\x89HDF\r\n\x1a\n", "signature"
        assert self.b[8] == 0 and self.b[13] == 8 and self.b[14] == 8, "superblock v0 with 8-byte offsets/lengths"
        self.leaf_k, self.int_k = struct.unpack_from("<HH", self.b, 16)
        base, fs, self.eof, drv = struct.unpack_from("<QQQQ", self.b, 24)
        assert base == 0 and fs == UNDEF and drv == UNDEF and self.eof == len(self.b), (self.eof, len(self.b))
        name_off, self.root_hdr, cache, _, bt, hp = struct.unpack_from("<QQIIQQ", self.b, 56)
        assert cache == 1
        self.root_cache = (bt, hp)

    def messages(self, addr):
        ver, _, nmsg, refc, size = struct.unpack_from("<BBHII", self.b, addr)
        assert ver == 1 and addr % 8 == 0
        out, blocks = [], [(addr + 16, size)]
        while blocks:
            a, n = blocks.pop(0)
            p = a
            while p + 8 <= a + n:
                t, sz, flags = struct.unpack_from("<HHB", self.b, p)
                assert sz % 8 == 0
                body = self.b[p + 8:p + 8 + sz]
                if t == 0x10:
                    blocks.append(struct.unpack_from("<QQ", body))
                elif t != 0:
                    out.append((t, body))
                p += 8 + sz
        assert len(out) <= nmsg
        return out

    def group(self, hdr):
        links = {}
        for t, body in self.messages(hdr):
            if t == 0x11:
                bt, hp = struct.unpack_from("<QQ", body)
                assert self.b[hp:hp + 4] == b"HEAP"
                dsize, free, daddr = struct.unpack_from("<QQQ", self.b, hp + 8)
                assert free == 1
                self._walk(bt, daddr, links, None)
        return links

    def _name(self, daddr, off):
        e = self.b.index(b"\0", daddr + off)
        return self.b[daddr + off:e].decode()

    def _walk(self, node, daddr, links, bound):
        sig = self.b[node:node + 4]
        if sig == b"SNOD":
            ver, _, n = struct.unpack_from("<BBH", self.b, node + 4)
            names = []
            for i in range(n):
                off, hdr, cache = struct.unpack_from("<QQI", self.b, node + 8 + 40 * i)
                names.append(self._name(daddr, off))
                links[names[-1]] = hdr
            assert names == sorted(names, key=lambda s: s.encode()), "symbol node entries must be sorted"
            if bound is not None:
                lo, hi = bound
                assert all(lo.encode() < x.encode() <= hi.encode() for x in names), (lo, hi, names[:3])
            return
        assert sig == b"TREE"
        ntype, level, used = struct.unpack_from("<BBH", self.b, node + 4)
        assert ntype == 0
        p = node + 24
        keys, kids = [], []
        for i in range(used):
            keys.append(struct.unpack_from("<Q", self.b, p)[0]); p += 8
            kids.append(struct.unpack_from("<Q", self.b, p)[0]); p += 8
        keys.append(struct.unpack_from("<Q", self.b, p)[0])
        for i, c in enumerate(kids):
            self._walk(c, daddr, links, (self._name(daddr, keys[i]), self._name(daddr, keys[i + 1])))

    def attrs(self, hdr):
        out = {}
        for t, body in self.messages(hdr):
            if t != 0x0C:
                continue
            ver, _, nsz, dtsz, dssz = struct.unpack_from("<BBHHH", body)
            assert ver == 1
            p = 8
            name = body[p:p + nsz].split(b"\0")[0].decode(); p += (nsz + 7) // 8 * 8
            dt = body[p:p + dtsz]; p += (dtsz + 7) // 8 * 8
            ds = body[p:p + dssz]; p += (dssz + 7) // 8 * 8
            assert ds[0] == 1 and ds[1] == 0, "scalar dataspace"
            cls = dt[0] & 15
            if cls == 9:
                assert dt[1] & 15 == 1 and dt[2] & 15 == 1, "vlen UTF-8 string"
                ln, gaddr, gidx = struct.unpack_from("<IQI", body, p)
                out[name] = self._gheap(gaddr, gidx)[:ln].decode()
            elif cls == 0:
                out[name] = struct.unpack_from("<q", body, p)[0]
        return out

    def _gheap(self, addr, idx):
        assert self.b[addr:addr + 4] == b"GCOL" and self.b[addr + 4] == 1
        size = struct.unpack_from("<Q", self.b, addr + 8)[0]
        assert size >= 4096
        p = addr + 16
        while p + 16 <= addr + size:
            i, ref, _, sz = struct.unpack_from("<HHIQ", self.b, p)
            if i == 0:
                assert p + sz == addr + size, "free-space object must span the rest of the collection"
                break
            if i == idx:
                return self.b[p + 16:p + 16 + sz]
            p += 16 + (sz + 7) // 8 * 8
        raise KeyError(idx)

    def dataset(self, hdr):
        dims = dtype = None
        layout = None
        deflate = False
        shuffle = 0
        for t, body in self.messages(hdr):
            if t == 1:
                assert body[0] == 1
                dims = struct.unpack_from("<%dQ" % body[1], body, 8)
            elif t == 3:
                cls, size = body[0] & 15, struct.unpack_from("<I", body, 4)[0]
                if cls == 1:
                    assert size == 2 and body[1] == 0x20 and body[2] == 15
                    off, prec, eloc, esz, mloc, msz, bias = struct.unpack_from("<HHBBBBI", body, 8)
                    assert (off, prec, eloc, esz, mloc, msz, bias) == (0, 16, 10, 5, 0, 10, 15)
                    dtype = np.float16
                else:
                    assert cls == 0 and size == 4 and body[1] & 8 == 0
                    dtype = np.uint32
            elif t == 8:
                assert body[0] == 3 and body[1] == 2
                rank1 = body[2]
                bt = struct.unpack_from("<Q", body, 3)[0]
                cd = struct.unpack_from("<%dI" % rank1, body, 11)
                layout = (bt, cd)
            elif t == 0x0B:
                assert body[0] == 1 and body[1] in (1, 2)
                p = 8
                for _ in range(body[1]):            # filters in the order they are applied on write
                    fid, nlen, flags, ncd = struct.unpack_from("<HHHH", body, p)
                    assert nlen == 0 and ncd == 1
                    val = struct.unpack_from("<I", body, p + 8)[0]
                    p += 16                         # header 8 + one client value 4 + padding 4
                    if fid == 2:
                        assert not deflate, "shuffle comes before deflate"
                        shuffle = val               # element size
                    else:
                        assert fid == 1
                        deflate = True
        bt, cd = layout
        assert cd[:2] == tuple(dims) and cd[2] == np.dtype(dtype).itemsize and deflate
        assert self.b[bt:bt + 4] == b"TREE" and self.b[bt + 4] == 1 and self.b[bt + 5] == 0
        used = struct.unpack_from("<H", self.b, bt + 6)[0]
        assert used == 1
        csize, mask, o0, o1, o2, child = struct.unpack_from("<IIQQQQ", self.b, bt + 24)
        assert (mask, o0, o1, o2) == (0, 0, 0, 0)
        raw = zlib.decompress(self.b[child:child + csize])
        if shuffle:
            assert shuffle == np.dtype(dtype).itemsize
            n = len(raw) // shuffle
            raw = np.frombuffer(raw, dtype=np.uint8).reshape(shuffle, n).T.tobytes()
        return np.frombuffer(raw, dtype=dtype).reshape(dims)
