"""Peer-to-peer KV connector: a prefill (producer) engine keeps the prefix blocks it has filled in host memory and serves them over
a socket; a decode (consumer) engine asks for blocks by their chained hashes and restores them instead of recomputing the prompt —
disaggregated prefill / decode without a shared file system.

Scheduler side (``P2pTier``, same interface as the other tiers): the producer turns every block that becomes full into a save
operation, the consumer's ``lookup`` asks the producer whether it holds a hash and ``restore`` turns a hit into a load operation.
Worker side: every producer rank runs a ``KVPageServer`` (ZMQ REP socket on ``port + rank``, LRU-bounded store of ``[layers][page]``
host tensors); a consumer rank fetches its own shard from the producer rank with the same index (``fetch_pages``).
Wire format: request ``[b"has", hash, ...]`` → ``[bitmap]``; ``[b"get", hash]`` → ``[json header, layer 0 bytes, layer 1 bytes, ...]``.
(reference: distributed/kv_transfer/kv_connector/v1/p2p/p2p_nccl_connector.py and p2p_nccl_engine.py: producer-side store,
consumer-side pull by request, roles kv_producer / kv_consumer)"""
from __future__ import annotations

import json
import threading
from collections import OrderedDict
from typing import Optional

import torch

SCHEME = "p2p://"


def handle_of(block_hash: bytes) -> str:
    return SCHEME + block_hash.hex()


def is_p2p(handle) -> bool:
    return isinstance(handle, str) and handle.startswith(SCHEME)


class P2pTier:
    def __init__(self, host: str, port: int, role: str) -> None:
        if role not in ("kv_producer", "kv_consumer"):
            raise ValueError("P2pConnector needs kv_role kv_producer or kv_consumer")
        self.host, self.port, self.role = host, port, role
        self.capacity = 1 << 62
        self.swap_out: list = []
        self.swap_in: list = []
        self.stored = self.restored = 0
        self._written: set = set()
        self._known: dict = {}      # consumer: hashes the producer confirmed
        self._sock = None

    # ---- producer
    def on_evict(self, block_hash: bytes, gpu_block: int) -> None:
        pass  # saved when the block became full

    def on_stored(self, block_hash: bytes, gpu_block: int) -> None:
        if self.role != "kv_producer" or block_hash in self._written:
            return
        self._written.add(block_hash)
        self.swap_out.append((gpu_block, handle_of(block_hash)))
        self.stored += 1

    # ---- consumer
    def _request(self, frames: list) -> Optional[list]:
        import zmq
        if self._sock is None:
            self._sock = zmq.Context.instance().socket(zmq.REQ)
            self._sock.setsockopt(zmq.LINGER, 0)
            self._sock.setsockopt(zmq.RCVTIMEO, 2000)
            self._sock.setsockopt(zmq.SNDTIMEO, 2000)
            self._sock.connect(f"tcp://{self.host}:{self.port}")
        try:
            self._sock.send_multipart(frames)
            return self._sock.recv_multipart()
        except zmq.ZMQError:
            self._sock.close()      # a REQ socket that missed its reply cannot be reused: the producer is treated as absent
            self._sock = None
            return None

    def lookup(self, block_hash: bytes):
        if self.role != "kv_consumer":
            return None
        if block_hash not in self._known:
            rep = self._request([b"has", block_hash])
            self._known[block_hash] = bool(rep and rep[0] and rep[0][0] == 1)
            if not self._known[block_hash]:
                del self._known[block_hash]     # it may arrive later: ask again next time
                return None
        return handle_of(block_hash)

    def restore(self, handle, gpu_block: int) -> None:
        self.swap_in.append((handle, gpu_block))
        self.restored += 1

    def take_ops(self) -> tuple[list, list]:
        out, inn = self.swap_out, self.swap_in
        self.swap_out, self.swap_in = [], []
        return out, inn

    def reset(self) -> None:
        self.swap_out, self.swap_in = [], []


class KVPageServer:
    """Producer rank: holds saved blocks and answers ``has`` / ``get`` until ``close()``."""

    def __init__(self, host: str, port: int, capacity_blocks: int = 4096) -> None:
        import zmq
        self.capacity = capacity_blocks
        self.store: OrderedDict = OrderedDict()
        self._lock = threading.Lock()
        self._sock = zmq.Context.instance().socket(zmq.REP)
        self._sock.setsockopt(zmq.LINGER, 0)
        self._sock.setsockopt(zmq.RCVTIMEO, 200)
        self._sock.bind(f"tcp://{host}:{port}")
        self._stop = False
        self._thread = threading.Thread(target=self._serve, daemon=True, name="onecat-kv-p2p")
        self._thread.start()

    def put(self, hash_hex: str, pages: list) -> None:
        with self._lock:
            self.store[hash_hex] = pages
            self.store.move_to_end(hash_hex)
            while len(self.store) > self.capacity:
                self.store.popitem(last=False)

    def _serve(self) -> None:
        import zmq
        while not self._stop:
            try:
                fr = self._sock.recv_multipart()
            except zmq.Again:
                continue
            except zmq.ZMQError:
                return
            if fr[0] == b"has":
                with self._lock:
                    rep = [bytes(1 if h.hex() in self.store else 0 for h in fr[1:])]
            elif fr[0] == b"get":
                with self._lock:
                    pages = self.store.get(fr[1].hex())
                    if pages is not None:
                        self.store.move_to_end(fr[1].hex())
                if pages is None:
                    rep = [b"{}"]
                else:
                    hdr = [{"dtype": str(p.dtype).replace("torch.", ""), "shape": list(p.shape)} for p in pages]
                    rep = [json.dumps(hdr).encode()] + [p.contiguous().view(torch.uint8).numpy().tobytes() for p in pages]
            else:
                rep = [b""]
            self._sock.send_multipart(rep)

    def close(self) -> None:
        self._stop = True
        self._thread.join(1.0)
        self._sock.close()


_FETCH = {}


def fetch_pages(host: str, port: int, hash_hex: str) -> Optional[list]:
    """Consumer rank: the ``[layers][page]`` tensors of one block from the producer rank listening on ``port``, or None."""
    import zmq
    key = (host, port)
    s = _FETCH.get(key)
    if s is None:
        s = zmq.Context.instance().socket(zmq.REQ)
        s.setsockopt(zmq.LINGER, 0)
        s.setsockopt(zmq.RCVTIMEO, 5000)
        s.setsockopt(zmq.SNDTIMEO, 5000)
        s.connect(f"tcp://{host}:{port}")
        _FETCH[key] = s
    try:
        s.send_multipart([b"get", bytes.fromhex(hash_hex)])
        fr = s.recv_multipart()
    except zmq.ZMQError:
        s.close()
        _FETCH.pop(key, None)
        return None
    hdr = json.loads(fr[0])
    if not hdr:
        return None
    out = []
    for h, raw in zip(hdr, fr[1:]):
        dt = getattr(torch, h["dtype"])
        out.append(torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dt).reshape(h["shape"]))
    return out
