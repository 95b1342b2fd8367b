"""Remote artifact cache: `http(s)://`, `s3://`, `gs://` (`gcs://`) URIs are fetched once into `$SUMMA_CACHE`
(default `~/.summa-cache`) and reused; `file://` and plain paths pass through.

Behaviour of `summa-llm/src/remote.rs:41-168,200-264`: the object's size comes from a HEAD, the body from exact
16 MiB ranged GETs written to a `.part` file that is synced and renamed into place, so a cache entry is either
absent or whole; the cache file name is a hash of the full URI plus the last path segment (never the query, so a
signed URL's secret does not reach the file system); messages show the URI without user info, query or fragment.

Object stores sit behind one small interface (`head(path) -> size`, `get_range(path, start, end) -> bytes`):
  * `HttpStore`: plain HTTP(S);
  * `S3Store`: virtual-hosted or endpoint-style requests signed with AWS Signature Version 4 from
    `AWS_ACCESS_KEY_ID` / `AWS_SECRET_ACCESS_KEY` (/ `AWS_SESSION_TOKEN`), region from `AWS_REGION` /
    `AWS_DEFAULT_REGION`, `AWS_ENDPOINT_URL` for S3-compatible stores; anonymous when no key is set;
  * `GcsStore`: the JSON API's media download with a bearer token from `GOOGLE_OAUTH_ACCESS_TOKEN`
    (or `SUMMA_GCS_TOKEN_COMMAND`, e.g. `gcloud auth print-access-token`); anonymous for public objects.
Every transport call goes through an injectable `opener(request) -> response`, which is how the tests run."""
from __future__ import annotations

import datetime
import hashlib
import hmac
import os
import re
import subprocess
import urllib.error
import urllib.parse
import urllib.request
from typing import Callable, Dict, Iterator, Optional, Tuple

CHUNK = 16 * 1024 * 1024
_SCHEMES = (("s3://", "s3"), ("gs://", "gs"), ("gcs://", "gs"), ("http://", "http"), ("https://", "https"))
_EMPTY_SHA = hashlib.sha256(b"").hexdigest()


class RemoteError(RuntimeError):
    pass


def remote_scheme(uri: str) -> Optional[str]:
    head = (uri or "")[:8].lower()
    return next((name for prefix, name in _SCHEMES if head.startswith(prefix)), None)


def redact(uri: str) -> str:
    """The URI without user info, query or fragment."""
    try:
        u = urllib.parse.urlsplit(uri)
        host = u.hostname or ""
        if u.port:
            host += f":{u.port}"
        if not u.scheme or not host:
            return "<invalid remote URI>"
        return urllib.parse.urlunsplit((u.scheme, host, u.path, "", ""))
    except ValueError:
        return "<invalid remote URI>"


def cache_dir() -> str:
    return os.environ.get("SUMMA_CACHE") or os.path.join(os.path.expanduser("~"), ".summa-cache")


def cache_file_name(uri: str) -> str:
    path = urllib.parse.urlsplit(uri).path
    segments = [s for s in path.split("/") if s]
    name = segments[-1] if segments and len(segments[-1]) <= 160 else "artifact"
    return hashlib.sha256(uri.encode()).hexdigest()[:32] + "-" + name


def ranges(size: int) -> Iterator[Tuple[int, int]]:
    """Half-open byte ranges that cover an object of `size` bytes exactly once."""
    return ((start, min(start + CHUNK, size)) for start in range(0, size, CHUNK))


# ------------------------------------------------------------------------------------------------ stores
class HttpStore:
    def __init__(self, opener: Optional[Callable] = None):
        self.opener = opener or urllib.request.urlopen

    def _headers(self, method: str, url: str, extra: Dict[str, str]) -> Dict[str, str]:
        return extra

    def _call(self, method: str, url: str, extra: Dict[str, str]):
        req = urllib.request.Request(url, method=method, headers=self._headers(method, url, extra))
        return self.opener(req)

    def url(self, path: str) -> str:
        return path

    def head(self, path: str) -> int:
        with self._call("HEAD", self.url(path), {}) as r:
            size = r.headers.get("Content-Length")
        if size is None:
            raise RemoteError("the server did not report an object size")
        return int(size)

    def get_range(self, path: str, start: int, end: int) -> bytes:
        with self._call("GET", self.url(path), {"Range": f"bytes={start}-{end - 1}"}) as r:
            data = r.read()
        if len(data) != end - start:
            raise RemoteError(f"ranged GET returned {len(data)} bytes for a {end - start}-byte range")
        return data


class S3Store(HttpStore):
    def __init__(self, bucket: str, opener: Optional[Callable] = None, env: Optional[Dict[str, str]] = None,
                 now: Optional[Callable[[], datetime.datetime]] = None):
        super().__init__(opener)
        env = os.environ if env is None else env
        self.bucket = bucket
        self.key_id, self.secret, self.token = env.get("AWS_ACCESS_KEY_ID"), env.get("AWS_SECRET_ACCESS_KEY"), env.get("AWS_SESSION_TOKEN")
        self.region = env.get("AWS_REGION") or env.get("AWS_DEFAULT_REGION") or "us-east-1"
        self.endpoint = (env.get("AWS_ENDPOINT_URL") or "").rstrip("/")
        self.now = now or (lambda: datetime.datetime.now(datetime.timezone.utc))

    def url(self, path: str) -> str:
        key = urllib.parse.quote(path.lstrip("/"), safe="/-_.~")
        if self.endpoint:
            return f"{self.endpoint}/{self.bucket}/{key}"
        host = f"{self.bucket}.s3.amazonaws.com" if self.region == "us-east-1" else f"{self.bucket}.s3.{self.region}.amazonaws.com"
        return f"https://{host}/{key}"

    def _headers(self, method: str, url: str, extra: Dict[str, str]) -> Dict[str, str]:
        if not (self.key_id and self.secret):
            return extra                                   # public bucket
        return sigv4_headers(method, url, extra, self.key_id, self.secret, self.token, self.region, "s3", self.now())


def sigv4_headers(method: str, url: str, headers: Dict[str, str], key_id: str, secret: str, token: Optional[str], region: str,
                  service: str, when: datetime.datetime) -> Dict[str, str]:
    """AWS Signature Version 4 for a request without a body: the given headers plus `host`, `x-amz-date`,
    `x-amz-content-sha256` (and the session token) are signed; returns the headers to send."""
    u = urllib.parse.urlsplit(url)
    amz_date, day = when.strftime("%Y%m%dT%H%M%SZ"), when.strftime("%Y%m%d")
    out = dict(headers)
    out.update({"Host": u.netloc, "x-amz-date": amz_date, "x-amz-content-sha256": _EMPTY_SHA})
    if token:
        out["x-amz-security-token"] = token
    signed = sorted((k.lower(), " ".join(v.split())) for k, v in out.items())
    names = ";".join(k for k, _ in signed)
    query = "&".join(sorted(f"{urllib.parse.quote(k, safe='-_.~')}={urllib.parse.quote(v, safe='-_.~')}"
                            for k, v in urllib.parse.parse_qsl(u.query, keep_blank_values=True)))
    canonical = "\n".join([method, u.path or "/", query, "".join(f"{k}:{v}\n" for k, v in signed), names, _EMPTY_SHA])
    scope = f"{day}/{region}/{service}/aws4_request"
    to_sign = "\n".join(["AWS4-HMAC-SHA256", amz_date, scope, hashlib.sha256(canonical.encode()).hexdigest()])
    key = ("AWS4" + secret).encode()
    for part in (day, region, service, "aws4_request"):
        key = hmac.new(key, part.encode(), hashlib.sha256).digest()
    signature = hmac.new(key, to_sign.encode(), hashlib.sha256).hexdigest()
    out["Authorization"] = f"AWS4-HMAC-SHA256 Credential={key_id}/{scope},SignedHeaders={names},Signature={signature}"
    return out


class GcsStore(HttpStore):
    def __init__(self, bucket: str, opener: Optional[Callable] = None, env: Optional[Dict[str, str]] = None, run: Optional[Callable] = None):
        super().__init__(opener)
        env = os.environ if env is None else env
        self.bucket = bucket
        self.bearer = env.get("GOOGLE_OAUTH_ACCESS_TOKEN")
        command = env.get("SUMMA_GCS_TOKEN_COMMAND")
        if not self.bearer and command:
            run = run or (lambda cmd: subprocess.run(cmd, shell=True, capture_output=True, text=True, timeout=60))
            done = run(command)
            if done.returncode != 0 or not done.stdout.strip():
                raise RemoteError("the access-token command failed")          # its output may hold a secret: not shown
            self.bearer = done.stdout.strip()

    def url(self, path: str) -> str:
        obj = urllib.parse.quote(path.lstrip("/"), safe="")
        return f"https://storage.googleapis.com/storage/v1/b/{self.bucket}/o/{obj}?alt=media"

    def _headers(self, method: str, url: str, extra: Dict[str, str]) -> Dict[str, str]:
        return dict(extra, Authorization=f"Bearer {self.bearer}") if self.bearer else extra

    def head(self, path: str) -> int:
        # the JSON API reports the size in the object's metadata (a HEAD on the media URL has no length)
        import json
        meta_url = self.url(path).replace("?alt=media", "?fields=size")
        with self._call("GET", meta_url, {}) as r:
            return int(json.loads(r.read())["size"])


def store_for(uri: str, opener: Optional[Callable] = None, env: Optional[Dict[str, str]] = None):
    """(store, path inside the store) of a remote URI."""
    scheme = remote_scheme(uri)
    if scheme in ("http", "https"):
        return HttpStore(opener), uri
    rest = uri.split("://", 1)[1]
    bucket, _, key = rest.partition("/")
    if not bucket or not key:
        raise RemoteError(f"{redact(uri)} does not name an object")
    key = key.split("?", 1)[0].split("#", 1)[0]
    return (S3Store(bucket, opener, env) if scheme == "s3" else GcsStore(bucket, opener, env)), key


# ------------------------------------------------------------------------------------------------ resolve
def resolve(uri: str, opener: Optional[Callable] = None, env: Optional[Dict[str, str]] = None) -> str:
    """Local path for `uri`, downloading it into the cache when it is remote."""
    if remote_scheme(uri) is None:
        return uri[7:] if (uri or "").startswith("file://") else uri
    dst = os.path.join(cache_dir(), cache_file_name(uri))
    if os.path.exists(dst):
        return dst
    os.makedirs(cache_dir(), exist_ok=True)
    part = dst + ".part"
    try:
        store, path = store_for(uri, opener, env)
        size = store.head(path)
        with open(part, "wb") as f:
            for start, end in ranges(size):
                f.write(store.get_range(path, start, end))
            f.flush()
            os.fsync(f.fileno())
        os.replace(part, dst)
    except Exception as e:
        if os.path.exists(part):
            os.unlink(part)
        detail = f"HTTP {e.code}" if isinstance(e, urllib.error.HTTPError) else (str(e) if isinstance(e, RemoteError) else type(e).__name__)
        raise RemoteError(f"fetching {redact(uri)} failed: {detail}") from None
    return dst
