"""TCP streams, listeners and the length-prefixed message framing used by the training-session remote control.

Parity: Source/Public/Oa/Network/Tcp.h (OaTcpStream: Connect / Read / Write / WriteAll / Close / RemoteAddr / RemotePort,
OaTcpListener: Bind / Accept / Port) and Network/TcpFramed.h (a message is a 4-byte little-endian length followed by
the payload).  Rendezvous inside this framework goes through the process group; this transport is for tools that talk
to a running job (pause / resume / checkpoint commands, metric streams).
"""
from __future__ import annotations

import socket
import struct
from typing import Optional, Tuple

from ..core.types import OaStatus, OaStatusCode

MAX_MESSAGE_BYTES = 256 << 20


class OaTcpStream:
    def __init__(self, sock: Optional[socket.socket] = None, addr: str = "", port: int = 0):
        self._s, self._addr, self._port = sock, addr, port

    @staticmethod
    def Connect(host: str, port: int, timeout: Optional[float] = 10.0) -> Tuple[Optional["OaTcpStream"], OaStatus]:
        try:
            s = socket.create_connection((host, port), timeout=timeout)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            s.settimeout(None)
        except OSError as e:
            return None, OaStatus(OaStatusCode.Unavailable, f"connect {host}:{port}: {e}")
        return OaTcpStream(s, host, port), OaStatus.Ok()

    def IsOpen(self) -> bool: return self._s is not None
    def NativeHandle(self) -> int: return self._s.fileno() if self._s is not None else -1
    def RemoteAddr(self) -> str: return self._addr
    def RemotePort(self) -> int: return self._port

    def Read(self, size: int) -> bytes:
        """Up to `size` bytes; empty when the peer closed."""
        if self._s is None:
            return b""
        try:
            return self._s.recv(size)
        except OSError:
            return b""

    def ReadExact(self, size: int) -> Optional[bytes]:
        buf = bytearray()
        while len(buf) < size:
            chunk = self.Read(size - len(buf))
            if not chunk:
                return None
            buf += chunk
        return bytes(buf)

    def Write(self, data: bytes) -> int:
        if self._s is None:
            return -1
        try:
            return self._s.send(data)
        except OSError:
            return -1

    def WriteAll(self, data: bytes) -> int:
        if self._s is None:
            return -1
        try:
            self._s.sendall(data)
            return len(data)
        except OSError:
            return -1

    def Close(self) -> None:
        if self._s is not None:
            try:
                self._s.shutdown(socket.SHUT_RDWR)
            except OSError:
                pass
            self._s.close()
            self._s = None

    def __del__(self):
        self.Close()


class OaTcpListener:
    def __init__(self, sock: Optional[socket.socket] = None, port: int = 0):
        self._s, self._port = sock, port

    @staticmethod
    def Bind(port: int, host: str = "127.0.0.1", backlog: int = 128) -> Tuple[Optional["OaTcpListener"], OaStatus]:
        """Port 0 lets the system choose; `Port()` reports the choice."""
        try:
            s = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            s.bind((host, port))
            s.listen(backlog)
        except OSError as e:
            return None, OaStatus(OaStatusCode.Unavailable, f"bind {host}:{port}: {e}")
        return OaTcpListener(s, s.getsockname()[1]), OaStatus.Ok()

    def IsOpen(self) -> bool: return self._s is not None
    def Port(self) -> int: return self._port

    def Accept(self, timeout: Optional[float] = None) -> Tuple[Optional[OaTcpStream], OaStatus]:
        if self._s is None:
            return None, OaStatus(OaStatusCode.FailedPrecondition, "listener is closed")
        try:
            self._s.settimeout(timeout)
            c, (addr, port) = self._s.accept()
            c.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        except socket.timeout:
            return None, OaStatus(OaStatusCode.DeadlineExceeded, "accept timed out")
        except OSError as e:
            return None, OaStatus(OaStatusCode.Unavailable, str(e))
        return OaTcpStream(c, addr, port), OaStatus.Ok()

    def Close(self) -> None:
        if self._s is not None:
            self._s.close()
            self._s = None

    def __del__(self):
        self.Close()


class OaTcpFramed:
    @staticmethod
    def WriteU32Le(value: int) -> bytes:
        return struct.pack("<I", value & 0xFFFFFFFF)

    @staticmethod
    def ReadU32Le(buf: bytes) -> Optional[int]:
        return struct.unpack("<I", buf[:4])[0] if len(buf) >= 4 else None

    @staticmethod
    def WriteMessage(stream: OaTcpStream, payload: bytes) -> OaStatus:
        if len(payload) > MAX_MESSAGE_BYTES:
            return OaStatus(OaStatusCode.InvalidArgument, "message larger than the framing limit")
        data = OaTcpFramed.WriteU32Le(len(payload)) + bytes(payload)
        return OaStatus.Ok() if stream.WriteAll(data) == len(data) else OaStatus(OaStatusCode.Unavailable, "connection lost while writing")

    @staticmethod
    def ReadMessage(stream: OaTcpStream) -> Tuple[Optional[bytes], OaStatus]:
        head = stream.ReadExact(4)
        if head is None:
            return None, OaStatus(OaStatusCode.Unavailable, "connection closed")
        n = OaTcpFramed.ReadU32Le(head)
        if n > MAX_MESSAGE_BYTES:
            return None, OaStatus(OaStatusCode.DataLoss, f"frame announces {n} bytes, beyond the framing limit")
        body = stream.ReadExact(n) if n else b""
        if body is None:
            return None, OaStatus(OaStatusCode.DataLoss, "connection closed inside a frame")
        return body, OaStatus.Ok()
