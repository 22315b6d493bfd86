"""Persistent stores behind the data layer: an ordered byte-key store, an embedded SQL store and the OHLCV store.

Parity: Source/Public/Oa/Data/KvStore.h (OaIKeyValueStore: Open / Close / Get / Put / Delete), Data/SqlStore.h
(CompactStorage / ExecuteSQL), Data/OhlcvStore.h (LoadData / LoadRecords / SaveData / SaveRecords / ticker
combinations / timestamps / counts / DeleteData), Data/StoreKind.h.  The reference binds RocksDB and DuckDB; neither is
part of this build, so the ordered store is an append-only log with a sorted in-memory index (CRC-checked records,
tombstones, compaction) and the SQL stores sit on the sqlite3 module of the standard library.
"""
from __future__ import annotations

import bisect
import enum
import os
import sqlite3
import struct
import zlib
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Tuple

from ..core.types import OaStatus, OaStatusCode
from .dataframe import OaDataOhlcv, OaRecordOhlcv


class OaStoreKind(enum.IntEnum):
    KvOrdered = 0
    SqlEmbedded = 1
    Composite = 2


_REC = struct.Struct("<IIiI")          # crc32, key length, value length (-1 = tombstone), reserved
_MAGIC = b"OAKV0001"


class OaKeyValueStore:
    """Byte keys -> byte values, ordered iteration.  Every Put / Delete appends one record; Open replays the log and
    stops at the first record whose checksum does not match (a torn tail after a crash is dropped, not fatal)."""

    def __init__(self):
        self._f = None
        self._path = ""
        self._ro = False
        self._index: Dict[bytes, Tuple[int, int]] = {}     # key -> (value offset, value length)
        self._keys: List[bytes] = []
        self._dead = 0

    def Kind(self) -> OaStoreKind: return OaStoreKind.KvOrdered
    def IsOpen(self) -> bool: return self._f is not None
    def IsReadOnly(self) -> bool: return self._ro
    def GetPath(self) -> str: return self._path

    def Open(self, path: str, read_only: bool = False) -> OaStatus:
        if self._f is not None:
            return OaStatus(OaStatusCode.FailedPrecondition, "store is already open")
        if read_only and not os.path.exists(path):
            return OaStatus(OaStatusCode.NotFound, f"{path} does not exist")
        fresh = not os.path.exists(path) or os.path.getsize(path) == 0
        self._f = open(path, "rb" if read_only else ("w+b" if fresh else "r+b"))
        self._path, self._ro = path, read_only
        self._index.clear(); self._dead = 0
        if fresh:
            self._f.write(_MAGIC); self._f.flush()
        else:
            if self._f.read(8) != _MAGIC:
                self._f.close(); self._f = None
                return OaStatus(OaStatusCode.DataLoss, f"{path} is not a key-value log")
            good = self._replay()
            if not read_only:
                self._f.truncate(good)
        self._keys = sorted(self._index)
        self._f.seek(0, os.SEEK_END)
        return OaStatus.Ok()

    def _replay(self) -> int:
        pos, size = 8, os.path.getsize(self._path)
        while pos + _REC.size <= size:
            self._f.seek(pos)
            crc, klen, vlen, _ = _REC.unpack(self._f.read(_REC.size))
            body_len = klen + max(vlen, 0)
            if pos + _REC.size + body_len > size:
                break
            body = self._f.read(body_len)
            if zlib.crc32(struct.pack("<Ii", klen, vlen) + body) != crc:
                break
            key = body[:klen]
            if key in self._index:
                self._dead += 1
            if vlen < 0:
                self._index.pop(key, None)
                self._dead += 1
            else:
                self._index[key] = (pos + _REC.size + klen, vlen)
            pos += _REC.size + body_len
        return pos

    def Close(self) -> None:
        if self._f is not None:
            self._f.close()
            self._f = None

    def _append(self, key: bytes, value: Optional[bytes]) -> int:
        vlen = -1 if value is None else len(value)
        body = key + (value or b"")
        self._f.seek(0, os.SEEK_END)
        pos = self._f.tell()
        self._f.write(_REC.pack(zlib.crc32(struct.pack("<Ii", len(key), vlen) + body), len(key), vlen, 0) + body)
        self._f.flush()
        return pos + _REC.size + len(key)

    def Put(self, key: bytes, value: bytes) -> OaStatus:
        if self._f is None or self._ro:
            return OaStatus(OaStatusCode.FailedPrecondition, "store is not open for writing")
        key, value = bytes(key), bytes(value)
        off = self._append(key, value)
        if key in self._index:
            self._dead += 1
        else:
            bisect.insort(self._keys, key)
        self._index[key] = (off, len(value))
        return OaStatus.Ok()

    def Get(self, key: bytes) -> Optional[bytes]:
        """The value, or None when the key is absent."""
        if self._f is None:
            return None
        hit = self._index.get(bytes(key))
        if hit is None:
            return None
        self._f.seek(hit[0])
        return self._f.read(hit[1])

    def Delete(self, key: bytes) -> OaStatus:
        if self._f is None or self._ro:
            return OaStatus(OaStatusCode.FailedPrecondition, "store is not open for writing")
        key = bytes(key)
        if key not in self._index:
            return OaStatus(OaStatusCode.NotFound, "key not found")
        self._append(key, None)
        del self._index[key]
        self._keys.pop(bisect.bisect_left(self._keys, key))
        self._dead += 2
        return OaStatus.Ok()

    def Count(self) -> int: return len(self._index)

    def Scan(self, start: bytes = b"", end: Optional[bytes] = None) -> Iterator[Tuple[bytes, bytes]]:
        """Pairs with start <= key < end in key order."""
        i = bisect.bisect_left(self._keys, bytes(start))
        while i < len(self._keys) and (end is None or self._keys[i] < end):
            k = self._keys[i]
            yield k, self.Get(k)
            i += 1

    def CompactStorage(self) -> OaStatus:
        """Rewrite the log with live records only (temp file + rename)."""
        if self._f is None or self._ro:
            return OaStatus(OaStatusCode.FailedPrecondition, "store is not open for writing")
        live = [(k, self.Get(k)) for k in self._keys]
        tmp = self._path + ".compact"
        self._f.close()
        with open(tmp, "wb") as f:
            f.write(_MAGIC)
        self._f = open(tmp, "r+b")
        self._index.clear()
        for k, v in live:
            self._index[k] = (self._append(k, v), len(v))
        self._f.close()
        os.replace(tmp, self._path)
        self._f = open(self._path, "r+b")
        self._dead = 0
        return OaStatus.Ok()

    def DeadRecords(self) -> int: return self._dead


class OaSqlStore:
    """Single-file (or in-memory, path ':memory:') SQL database."""

    def __init__(self):
        self._db: Optional[sqlite3.Connection] = None
        self._path, self._ro = "", False

    def Kind(self) -> OaStoreKind: return OaStoreKind.SqlEmbedded
    def IsOpen(self) -> bool: return self._db is not None
    def IsReadOnly(self) -> bool: return self._ro
    def GetPath(self) -> str: return self._path

    def Open(self, path: str, read_only: bool = False) -> OaStatus:
        try:
            if read_only:
                self._db = sqlite3.connect(f"file:{path}?mode=ro", uri=True)
            else:
                self._db = sqlite3.connect(path)
        except sqlite3.Error as e:
            return OaStatus(OaStatusCode.Unavailable, str(e))
        self._path, self._ro = path, read_only
        return OaStatus.Ok()

    def Close(self) -> None:
        if self._db is not None:
            self._db.close()
            self._db = None

    def ExecuteSQL(self, query: str, params: tuple = ()) -> OaStatus:
        if self._db is None:
            return OaStatus(OaStatusCode.FailedPrecondition, "store is not open")
        try:
            with self._db:
                self._db.execute(query, params)
        except sqlite3.Error as e:
            return OaStatus(OaStatusCode.InvalidArgument, str(e))
        return OaStatus.Ok()

    def Query(self, query: str, params: tuple = ()) -> List[tuple]:
        if self._db is None:
            raise RuntimeError("store is not open")
        return self._db.execute(query, params).fetchall()

    def CompactStorage(self) -> OaStatus:
        return self.ExecuteSQL("VACUUM") if not self._ro else OaStatus(OaStatusCode.FailedPrecondition, "read-only store")


@dataclass
class OaContractTicker:
    Ticker: str
    ContractType: str
    Interval: str


@dataclass
class OaDataSummary:
    Ticker: str
    ContractType: str
    Interval: str
    Count: int
    Earliest: float
    Latest: float


class OaOhlcvStore(OaSqlStore):
    """Bars keyed by (ticker, contract type, interval, time); saving a bar that exists replaces it."""

    _TABLE = ("CREATE TABLE IF NOT EXISTS ohlcv (ticker TEXT NOT NULL, contract TEXT NOT NULL, interval TEXT NOT NULL, time REAL NOT NULL, "
              "open REAL, high REAL, low REAL, close REAL, volume REAL, PRIMARY KEY (ticker, contract, interval, time))")

    def Open(self, path: str, read_only: bool = False) -> OaStatus:
        st = super().Open(path, read_only)
        if st.IsOk() and not read_only:
            st = self.ExecuteSQL(self._TABLE)
        return st

    @staticmethod
    def _range(start: Optional[float], end: Optional[float]) -> Tuple[str, tuple]:
        sql, args = "", ()
        if start is not None:
            sql, args = sql + " AND time >= ?", args + (float(start),)
        if end is not None:
            sql, args = sql + " AND time <= ?", args + (float(end),)
        return sql, args

    def SaveRecords(self, ticker: str, contract: str, interval: str, records: List[OaRecordOhlcv]) -> OaStatus:
        if self._db is None or self._ro:
            return OaStatus(OaStatusCode.FailedPrecondition, "store is not open for writing")
        bad = [r for r in records if not r.IsValid()]
        if bad:
            return OaStatus(OaStatusCode.InvalidArgument, f"{len(bad)} bar(s) with high below low / open / close")
        with self._db:
            self._db.executemany("INSERT OR REPLACE INTO ohlcv VALUES (?,?,?,?,?,?,?,?,?)",
                                 [(ticker, contract, interval, r.Time, r.Open, r.High, r.Low, r.Close, r.Volume) for r in records])
        return OaStatus.Ok()

    def SaveData(self, ticker: str, contract: str, interval: str, data: OaDataOhlcv) -> OaStatus:
        return self.SaveRecords(ticker, contract, interval, data.Records())

    def LoadRecords(self, ticker: str, contract: str, interval: str, start: Optional[float] = None,
                    end: Optional[float] = None) -> List[OaRecordOhlcv]:
        extra, args = self._range(start, end)
        rows = self.Query("SELECT time, open, high, low, close, volume FROM ohlcv WHERE ticker=? AND contract=? AND interval=?" + extra +
                          " ORDER BY time", (ticker, contract, interval) + args)
        return [OaRecordOhlcv(*r) for r in rows]

    def LoadData(self, ticker: str, contract: str, interval: str, start: Optional[float] = None, end: Optional[float] = None) -> OaDataOhlcv:
        return OaDataOhlcv(self.LoadRecords(ticker, contract, interval, start, end))

    def GetTickerCombinations(self) -> List[OaContractTicker]:
        return [OaContractTicker(*r) for r in self.Query("SELECT DISTINCT ticker, contract, interval FROM ohlcv ORDER BY 1, 2, 3")]

    def GetAvailableData(self) -> List[OaDataSummary]:
        return [OaDataSummary(*r) for r in self.Query(
            "SELECT ticker, contract, interval, COUNT(*), MIN(time), MAX(time) FROM ohlcv GROUP BY 1, 2, 3 ORDER BY 1, 2, 3")]

    def _agg(self, fn: str, ticker: str, contract: str, interval: str):
        return self.Query(f"SELECT {fn} FROM ohlcv WHERE ticker=? AND contract=? AND interval=?", (ticker, contract, interval))[0][0]

    def GetEarliestTimestamp(self, ticker, contract, interval) -> Optional[float]: return self._agg("MIN(time)", ticker, contract, interval)
    def GetLatestTimestamp(self, ticker, contract, interval) -> Optional[float]: return self._agg("MAX(time)", ticker, contract, interval)
    def GetRecordCount(self, ticker, contract, interval) -> int: return int(self._agg("COUNT(*)", ticker, contract, interval))

    def GetAllTimestamps(self, ticker, contract, interval) -> List[float]:
        return [r[0] for r in self.Query("SELECT time FROM ohlcv WHERE ticker=? AND contract=? AND interval=? ORDER BY time",
                                         (ticker, contract, interval))]

    def DeleteData(self, ticker: str, contract: str, interval: str, start: Optional[float] = None, end: Optional[float] = None) -> OaStatus:
        extra, args = self._range(start, end)
        return self.ExecuteSQL("DELETE FROM ohlcv WHERE ticker=? AND contract=? AND interval=?" + extra, (ticker, contract, interval) + args)
