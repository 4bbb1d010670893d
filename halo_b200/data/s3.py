"""S3 object storage as a dataset and checkpoint location, without an SDK: requests signed with AWS Signature
Version 4 over plain HTTPS (``requests``), which is all that listing, reading, writing and deleting objects need.

``S3Client`` talks to AWS or to any S3-compatible endpoint (``endpoint_url``; path-style addressing there). Folder
transfers run on a thread pool, skip objects whose size and ETag already match the local copy's record, and write each
file through a temporary name so that an interrupted download never leaves a truncated shard behind.
``resolve_dataset_path`` turns an ``s3://bucket/prefix`` dataset path into a local directory: the first rank of a node
downloads into the cache, the others wait for its completion marker.

Credentials come from the arguments, else ``AWS_ACCESS_KEY_ID`` / ``AWS_SECRET_ACCESS_KEY`` / ``AWS_SESSION_TOKEN``;
region from ``AWS_DEFAULT_REGION`` (default ``us-east-1``).

Counterpart of halo/data/sources/s3_client.py:91-376 and halo/data/sources/s3_dataset_store.py (boto3 there).
"""

from __future__ import annotations

import concurrent.futures as cf
import datetime
import hashlib
import hmac
import json
import os
import time
import urllib.parse
import xml.etree.ElementTree as ET
from dataclasses import dataclass

EMPTY_SHA256 = hashlib.sha256(b"").hexdigest()
UNSIGNED = "UNSIGNED-PAYLOAD"


def _hmac(key: bytes, msg: str) -> bytes:
    return hmac.new(key, msg.encode(), hashlib.sha256).digest()


def _quote(s: str, safe: str = "-_.~") -> str:
    return urllib.parse.quote(s, safe=safe)


def sign_v4(method: str, host: str, path: str, query: dict, headers: dict, payload_hash: str, access_key: str, secret_key: str,
            region: str, amz_date: str, service: str = "s3") -> str:
    """The ``Authorization`` header value for one request. ``headers`` must already hold every header to sign (``host``,
    ``x-amz-date``, ``x-amz-content-sha256`` included); ``path`` is the URI-encoded absolute path."""
    canonical_query = "&".join(f"{_quote(k)}={_quote(str(v))}" for k, v in sorted(query.items()))
    lowered = {k.lower(): " ".join(str(v).split()) for k, v in headers.items()}
    signed = ";".join(sorted(lowered))
    canonical_headers = "".join(f"{k}:{lowered[k]}\n" for k in sorted(lowered))
    canonical = "\n".join([method, path, canonical_query, canonical_headers, signed, payload_hash])
    date = amz_date[:8]
    scope = f"{date}/{region}/{service}/aws4_request"
    to_sign = "\n".join(["AWS4-HMAC-SHA256", amz_date, scope, hashlib.sha256(canonical.encode()).hexdigest()])
    key = _hmac(_hmac(_hmac(_hmac(("AWS4" + secret_key).encode(), date), region), service), "aws4_request")
    signature = hmac.new(key, to_sign.encode(), hashlib.sha256).hexdigest()
    return f"AWS4-HMAC-SHA256 Credential={access_key}/{scope},SignedHeaders={signed},Signature={signature}"


def parse_s3_uri(uri: str) -> tuple[str, str]:
    if not uri.startswith("s3://"):
        raise ValueError(f"{uri!r} is not an s3:// URI")
    bucket, _, key = uri[5:].partition("/")
    if not bucket:
        raise ValueError(f"{uri!r} names no bucket")
    return bucket, key


@dataclass
class S3Object:
    key: str
    size: int
    etag: str


class S3Client:
    def __init__(self, bucket: str, region: str | None = None, access_key: str | None = None, secret_key: str | None = None,
                 session_token: str | None = None, endpoint_url: str | None = None, session=None, max_workers: int = 16,
                 retries: int = 4, timeout_s: float = 120.0):
        self.bucket = bucket
        self.region = region or os.environ.get("AWS_DEFAULT_REGION") or os.environ.get("AWS_REGION") or "us-east-1"
        self.access_key = access_key or os.environ.get("AWS_ACCESS_KEY_ID", "")
        self.secret_key = secret_key or os.environ.get("AWS_SECRET_ACCESS_KEY", "")
        self.session_token = session_token or os.environ.get("AWS_SESSION_TOKEN", "")
        self.endpoint_url = (endpoint_url or os.environ.get("AWS_ENDPOINT_URL_S3") or "").rstrip("/")
        self._session, self.max_workers, self.retries, self.timeout_s = session, max_workers, retries, timeout_s
        if not self.access_key or not self.secret_key:
            raise PermissionError("no S3 credentials: set AWS_ACCESS_KEY_ID and AWS_SECRET_ACCESS_KEY (or pass them)")

    # ---- one request ----------------------------------------------------------------------------------
    def _http(self):
        if self._session is None:
            import requests

            self._session = requests.Session()
        return self._session

    def _address(self, key: str) -> tuple[str, str, str]:
        """(url base, host header, URI-encoded path) - virtual-hosted style on AWS, path style on a custom endpoint."""
        enc = "/" + _quote(key, safe="-_.~/")
        if self.endpoint_url:
            host = self.endpoint_url.split("//", 1)[1]
            return self.endpoint_url, host, f"/{self.bucket}{enc}" if key else f"/{self.bucket}"
        host = f"{self.bucket}.s3.{self.region}.amazonaws.com"
        return f"https://{host}", host, enc if key else "/"

    def _request(self, method: str, key: str, query: dict | None = None, data=None, headers: dict | None = None, stream: bool = False,
                 ok=(200, 204, 206)):
        query = dict(query or {})
        base, host, path = self._address(key)
        payload_hash = UNSIGNED if data is not None and not isinstance(data, (bytes, bytearray)) else hashlib.sha256(data or b"").hexdigest()
        delay, last = 0.5, None
        for attempt in range(self.retries):
            now = datetime.datetime.now(datetime.timezone.utc).strftime("%Y%m%dT%H%M%SZ")
            signed = {"host": host, "x-amz-date": now, "x-amz-content-sha256": payload_hash, **(headers or {})}
            if self.session_token:
                signed["x-amz-security-token"] = self.session_token
            auth = sign_v4(method, host, path, query, signed, payload_hash, self.access_key, self.secret_key, self.region, now)
            send = {k: v for k, v in signed.items() if k != "host"}
            send["Authorization"] = auth
            qs = "&".join(f"{_quote(k)}={_quote(str(v))}" for k, v in sorted(query.items()))
            url = base + path + ("?" + qs if qs else "")
            try:
                resp = self._http().request(method, url, headers=send, data=data, stream=stream, timeout=self.timeout_s)
            except Exception as exc:  # noqa: BLE001 - connection errors are retried
                last = exc
            else:
                if resp.status_code in ok or resp.status_code == 404:
                    return resp
                last = RuntimeError(f"S3 {method} {self.bucket}/{key}: HTTP {resp.status_code} {resp.text[:300]}")
                if resp.status_code < 500 and resp.status_code not in (429,):
                    raise last
            if attempt + 1 < self.retries:
                time.sleep(delay)
                delay = min(delay * 2, 8.0)
        raise ConnectionError(f"S3 {method} {self.bucket}/{key} failed after {self.retries} attempts: {last}")

    # ---- objects --------------------------------------------------------------------------------------
    def object_exists(self, key: str) -> bool:
        return self._request("HEAD", key).status_code == 200

    def list_objects(self, prefix: str = "") -> list[S3Object]:
        out, token = [], None
        while True:
            query = {"list-type": "2", "prefix": prefix, "max-keys": "1000"}
            if token:
                query["continuation-token"] = token
            resp = self._request("GET", "", query=query)
            if resp.status_code == 404:
                raise FileNotFoundError(f"no bucket {self.bucket!r}")
            root = ET.fromstring(resp.content)
            ns = root.tag[:root.tag.index("}") + 1] if root.tag.startswith("{") else ""
            for c in root.findall(f"{ns}Contents"):
                out.append(S3Object(c.findtext(f"{ns}Key"), int(c.findtext(f"{ns}Size") or 0), (c.findtext(f"{ns}ETag") or "").strip('"')))
            if (root.findtext(f"{ns}IsTruncated") or "false").lower() != "true":
                return out
            token = root.findtext(f"{ns}NextContinuationToken")

    def exists(self, prefix: str) -> bool:
        """An object with this key, or any object below it as a folder."""
        return self.object_exists(prefix) or bool(self.list_objects(prefix.rstrip("/") + "/")[:1])

    def read_bytes(self, key: str) -> bytes:
        resp = self._request("GET", key)
        if resp.status_code == 404:
            raise FileNotFoundError(f"s3://{self.bucket}/{key}")
        return resp.content

    def write_bytes(self, key: str, data: bytes) -> None:
        self._request("PUT", key, data=bytes(data))

    def delete(self, key: str, recursive: bool = True) -> int:
        keys = [o.key for o in self.list_objects(key.rstrip("/") + "/")] if recursive else []
        if self.object_exists(key):
            keys.append(key)
        for k in keys:
            self._request("DELETE", k)
        return len(keys)

    def content_fingerprint(self, prefix: str) -> str | None:
        """A digest of (key, size, ETag) of everything under ``prefix``: changes when any object does."""
        objs = sorted(self.list_objects(prefix.rstrip("/") + "/"), key=lambda o: o.key)
        if not objs:
            return None
        h = hashlib.sha256()
        for o in objs:
            h.update(f"{o.key}\0{o.size}\0{o.etag}\n".encode())
        return h.hexdigest()

    # ---- folders --------------------------------------------------------------------------------------
    def download_file(self, key: str, path: str) -> int:
        resp = self._request("GET", key, stream=True)
        if resp.status_code == 404:
            raise FileNotFoundError(f"s3://{self.bucket}/{key}")
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        tmp = f"{path}.part{os.getpid()}"
        n = 0
        with open(tmp, "wb") as f:
            for block in resp.iter_content(1 << 22):
                f.write(block)
                n += len(block)
        os.replace(tmp, path)
        return n

    def download_folder(self, prefix: str, local_dir: str) -> dict:
        """Mirror everything under ``prefix`` into ``local_dir``; objects whose recorded size and ETag match are skipped."""
        prefix = prefix.rstrip("/") + "/" if prefix else ""
        objs = [o for o in self.list_objects(prefix) if not o.key.endswith("/")]
        if not objs:
            raise FileNotFoundError(f"nothing under s3://{self.bucket}/{prefix}")
        record_path = os.path.join(local_dir, ".s3_objects.json")
        have = json.load(open(record_path)) if os.path.isfile(record_path) else {}
        todo = [o for o in objs if have.get(o.key) != [o.size, o.etag] or not os.path.isfile(os.path.join(local_dir, o.key[len(prefix):]))]
        with cf.ThreadPoolExecutor(max_workers=self.max_workers) as pool:
            moved = sum(pool.map(lambda o: self.download_file(o.key, os.path.join(local_dir, o.key[len(prefix):])), todo))
        os.makedirs(local_dir, exist_ok=True)
        tmp = record_path + ".part"
        json.dump({o.key: [o.size, o.etag] for o in objs}, open(tmp, "w"))
        os.replace(tmp, record_path)
        return {"objects": len(objs), "downloaded": len(todo), "bytes": moved}

    def push_folder(self, local_dir: str, prefix: str) -> dict:
        prefix = prefix.rstrip("/") + "/" if prefix else ""
        files = []
        for root, _, names in os.walk(local_dir):
            for n in names:
                if n.startswith(".s3_objects") or ".part" in n:
                    continue
                full = os.path.join(root, n)
                files.append((full, prefix + os.path.relpath(full, local_dir).replace(os.sep, "/")))

        def put(item):
            full, key = item
            with open(full, "rb") as f:
                data = f.read()
            self.write_bytes(key, data)
            return len(data)

        with cf.ThreadPoolExecutor(max_workers=self.max_workers) as pool:
            moved = sum(pool.map(put, files))
        return {"objects": len(files), "bytes": moved}


def resolve_dataset_path(path: str, cache_root: str | None = None, client: S3Client | None = None, is_downloader: bool = True,
                         wait_timeout_s: float = 3600.0) -> str:
    """A local directory holding the dataset at ``path``. Local paths pass through; ``s3://bucket/prefix`` is mirrored into
    ``cache_root`` by the process with ``is_downloader`` (one per node); the others wait for its completion marker, which
    carries the remote content fingerprint so that a changed dataset is fetched again."""
    if not path.startswith("s3://"):
        return path
    bucket, prefix = parse_s3_uri(path)
    client = client or S3Client(bucket)
    cache_root = cache_root or os.path.join(os.environ.get("HALO_DATA_ROOT", os.path.expanduser("~/.cache/halo_b200")), "s3")
    local = os.path.join(cache_root, bucket, prefix.strip("/"))
    marker = os.path.join(local, ".complete")
    if is_downloader:
        fingerprint = client.content_fingerprint(prefix) or ""
        if not (os.path.isfile(marker) and open(marker).read().strip() == fingerprint):
            client.download_folder(prefix, local)
            tmp = marker + ".part"
            open(tmp, "w").write(fingerprint)
            os.replace(tmp, marker)
        return local
    deadline = time.monotonic() + wait_timeout_s
    while not os.path.isfile(marker):
        if time.monotonic() > deadline:
            raise TimeoutError(f"{local} was not downloaded within {wait_timeout_s:g} s by this node's first rank")
        time.sleep(1.0)
    return local
