"""Client of a remote attention daemon ("attnd"): attention of one layer is computed by a
server that owns the KV cache, reached with one UDP datagram per (token, kv head) carrying
the head's queries and the new K/V row (zml/attention/attnd.zig of the reference).

Wire format (little endian, packed; attnd.zig `Header`): ::

    u8  type ('a' attn, 's' start, 'p' ping)     u8  kv_head_id
    u64 conversation_id     u32 token_pos        u16 layer_id
    u8  model_id            u8  first_q_id       u8  num_queries
    u8  magic[3] = "ZML"

followed by `num_queries` query heads, one K row and one V row (bf16).  The reply repeats the
header and carries `num_queries` output heads.  Ethernet + IP + UDP + this header is a multiple
of 4 bytes, so payloads stay 4-byte aligned on the wire.

`Daemon` is a small in-process server with the same protocol (a KV store per conversation /
layer / head and causal softmax attention in float32); it is what the tests talk to over
loopback, and a reference for writing a real one.
"""
from __future__ import annotations

import enum
import socket
import struct
import threading
from dataclasses import dataclass
from typing import Optional

import torch

from ..tensor import Tensor

HEADER = struct.Struct("<BBQIHBBB3s")
MAGIC = b"ZML"
MAX_CONCURRENT_PACKETS_PER_CLIENT = 32
assert (14 + 20 + 8 + HEADER.size) % 4 == 0


class MessageType(enum.IntEnum):
    attn = ord("a")
    start = ord("s")
    ping = ord("p")


class ModelId(enum.IntEnum):
    llama_3_1_8b = 0
    llama_3_2_1b = 1
    qwen3_14b = 2
    qwen3_32b = 3


class AttndError(RuntimeError):
    pass


@dataclass
class Header:
    type: int
    kv_head_id: int
    conversation_id: int
    token_pos: int
    layer_id: int
    model_id: int
    first_q_id: int
    num_queries: int

    def pack(self) -> bytes:
        return HEADER.pack(self.type, self.kv_head_id, self.conversation_id, self.token_pos, self.layer_id,
                           self.model_id, self.first_q_id, self.num_queries, MAGIC)

    @staticmethod
    def parse(data: bytes) -> tuple["Header", bytes]:
        if len(data) < HEADER.size:
            raise AttndError("ShortMessage")
        *f, magic = HEADER.unpack_from(data)
        if magic != MAGIC:
            raise AttndError("InvalidHeader")
        return Header(*f), data[HEADER.size:]


@dataclass
class Config:
    destination: tuple          # (host, port)
    mtu: int = 1500
    timeout_s: float = 2.0


_context: Optional["Context"] = None


class Client:
    """One UDP socket (one per local device in the reference, attnd.zig:318-352)."""

    def __init__(self, config: Config):
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        self.sock.bind(("0.0.0.0", 0))
        size = config.mtu * MAX_CONCURRENT_PACKETS_PER_CLIENT
        self.sock.setsockopt(socket.SOL_SOCKET, socket.SO_RCVBUF, size)
        self.sock.setsockopt(socket.SOL_SOCKET, socket.SO_SNDBUF, size)
        self.sock.settimeout(config.timeout_s)
        self.destination = config.destination
        self.mtu = config.mtu

    def send(self, header: Header, q: bytes, k: bytes, v: bytes) -> None:
        pkt = header.pack() + q + k + v
        if len(pkt) > self.mtu:
            raise AttndError(f"datagram of {len(pkt)} bytes exceeds the MTU {self.mtu}")
        self.sock.sendto(pkt, self.destination)

    def receive(self) -> tuple[Header, bytes]:
        try:
            data, _ = self.sock.recvfrom(self.mtu)
        except socket.timeout as e:
            raise AttndError("no reply from the attention daemon") from e
        return Header.parse(data)

    def ping(self) -> bool:
        self.sock.sendto(Header(MessageType.ping, 0, 0, 0, 0, 0, 0, 0).pack(), self.destination)
        try:
            h, _ = self.receive()
        except AttndError:
            return False
        return h.type == MessageType.ping

    def close(self) -> None:
        self.sock.close()


class Context:
    def __init__(self, config: Config, num_devices: int = 1):
        self.mtu = config.mtu
        self.clients = [Client(config) for _ in range(num_devices)]

    def close(self) -> None:
        for c in self.clients:
            c.close()


def register(config: Config, num_devices: int = 1) -> Context:
    """Opens the sockets; must precede `Parameters.init` (which needs the MTU)."""
    global _context
    if _context is not None:
        _context.close()
    _context = Context(config, num_devices)
    return _context


def deinit() -> None:
    global _context
    if _context is not None:
        _context.close()
        _context = None


@dataclass
class Parameters:
    model_id: int
    head_dim: int
    head_bytes: int
    num_kv_heads: int
    num_q_per_head: int
    num_q_per_packet: int
    is_prefill: bool

    @staticmethod
    def init(model_id: int, head_dim: int, num_attention_heads: int, num_kv_heads: int, is_prefill: bool) -> "Parameters":
        if _context is None:
            raise AttndError("attnd wasn't registered yet, use register() first")
        mtu = _context.mtu
        num_q_per_head = num_attention_heads // num_kv_heads
        if num_q_per_head * num_kv_heads != num_attention_heads:
            raise ValueError("attention heads must be a multiple of kv heads")
        head_bytes = head_dim * 2                      # bf16 or another 16-bit type
        max_q = min((mtu - HEADER.size - 2 * head_bytes) // head_bytes, num_q_per_head)
        if max_q < 1:
            raise AttndError(f"MTU {mtu} cannot carry one query with its K/V row")
        packets = -(-num_q_per_head // max_q)
        while num_q_per_head % packets != 0:
            packets += 1
        return Parameters(int(model_id), head_dim, head_bytes, num_kv_heads, num_q_per_head, num_q_per_head // packets,
                          is_prefill)


@dataclass
class Metadata:
    conversation_id: int = 749
    layer_id: int = 0
    num_tokens: int = 0


def causal_attention(q: Tensor, k: Tensor, v: Tensor, token_offset, metadata: Metadata, parameters: Parameters,
                     device_ordinal: int = 0, num_partitions: int = 1, new_rows_only: bool = False) -> Tensor:
    """q {q, h, hd}; k, v {k, h, hd}.  In decode only the K/V row at `token_offset` is sent: `k` / `v` are the
    whole cache and the row is read at that index, or - with `new_rows_only` - they hold just the new row."""
    if _context is None:
        raise AttndError("attnd wasn't registered yet, use register() first")
    client = _context.clients[device_ordinal]
    p = parameters
    t0 = int(token_offset.to_torch().reshape(-1)[0]) if isinstance(token_offset, Tensor) else int(token_offset)
    qt = q.transpose(("q", "h", "hd")).to_torch().contiguous()
    kt = k.transpose(("k", "h", "hd")).to_torch()
    vt = v.transpose(("k", "h", "hd")).to_torch()
    n = metadata.num_tokens or qt.shape[0]
    if p.is_prefill:
        kt, vt = kt[:n], vt[:n]
    elif not new_rows_only:
        kt, vt = kt[t0:t0 + 1], vt[t0:t0 + 1]
    heads_local = p.num_kv_heads // num_partitions
    head0 = heads_local * device_ordinal
    raw = lambda t: t.contiguous().view(torch.int16).cpu().numpy().tobytes()
    out = torch.empty_like(qt, device="cpu")
    out_i16 = out.view(torch.int16)
    for t in range(n):
        sent = 0
        for h in range(heads_local):
            kb, vb = raw(kt[t, h]), raw(vt[t, h])
            first = 0
            while first < p.num_q_per_head:
                nq = min(p.num_q_per_head - first, p.num_q_per_packet)
                hdr = Header(MessageType.attn, head0 + h, metadata.conversation_id, t0 + t, metadata.layer_id,
                             p.model_id, first, nq)
                qh = qt[t, h * p.num_q_per_head + first:h * p.num_q_per_head + first + nq]
                client.send(hdr, raw(qh), kb, vb)
                first += nq
                sent += 1
        got = 0
        while got < heads_local * p.num_q_per_head:
            hdr, payload = client.receive()
            if hdr.num_queries > p.num_q_per_head or hdr.kv_head_id >= p.num_kv_heads or \
                    len(payload) != hdr.num_queries * p.head_bytes:
                raise AttndError("malformed reply")
            h = hdr.kv_head_id - head0
            rows = torch.frombuffer(bytearray(payload), dtype=torch.int16).view(hdr.num_queries, p.head_dim)
            tok = hdr.token_pos - t0
            out_i16[tok, h * p.num_q_per_head + hdr.first_q_id:h * p.num_q_per_head + hdr.first_q_id + hdr.num_queries] = rows
            got += hdr.num_queries
            sent -= 1
        if sent != 0:
            raise AttndError("reply count does not match the requests sent")
    res = out.to(qt.device)
    return Tensor(res, q.transpose(("q", "h", "hd")).shape()).transpose(q.shape().tags)


class Daemon:
    """Loopback attention server speaking the protocol above.  KV rows are stored per
    (conversation, layer, kv head) at `token_pos`; a request is answered with the causal softmax
    attention of its queries over rows 0..token_pos."""

    def __init__(self, host: str = "127.0.0.1", port: int = 0, mtu: int = 1500):
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        self.sock.bind((host, port))
        self.sock.settimeout(0.2)
        self.address = self.sock.getsockname()
        self.mtu = mtu
        self.kv: dict = {}
        self.requests = 0
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._serve, daemon=True)

    def start(self) -> "Daemon":
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2.0)
        self.sock.close()

    def _serve(self) -> None:
        while not self._stop.is_set():
            try:
                data, peer = self.sock.recvfrom(65536)
            except socket.timeout:
                continue
            except OSError:
                return
            try:
                hdr, payload = Header.parse(data)
            except AttndError:
                continue
            if hdr.type == MessageType.ping:
                self.sock.sendto(hdr.pack(), peer)
                continue
            if hdr.type == MessageType.start:
                for key in [k for k in self.kv if k[0] == hdr.conversation_id]:
                    del self.kv[key]
                continue
            self.requests += 1
            hb = (len(payload) // (hdr.num_queries + 2))
            hd = hb // 2
            buf = torch.frombuffer(bytearray(payload), dtype=torch.int16).view(torch.bfloat16).view(hdr.num_queries + 2, hd)
            qh, krow, vrow = buf[:hdr.num_queries].float(), buf[-2], buf[-1]
            store = self.kv.setdefault((hdr.conversation_id, hdr.layer_id, hdr.kv_head_id), {})
            store[hdr.token_pos] = (krow.clone(), vrow.clone())
            pos = [p for p in sorted(store) if p <= hdr.token_pos]
            ks = torch.stack([store[p][0] for p in pos]).float()
            vs = torch.stack([store[p][1] for p in pos]).float()
            w = torch.softmax(qh @ ks.t() / (hd ** 0.5), dim=-1)
            o = (w @ vs).to(torch.bfloat16).contiguous()
            self.sock.sendto(hdr.pack() + o.view(torch.int16).numpy().tobytes(), peer)
