"""Resolution of media references in requests (``data:`` URLs, ``http(s)://`` links, ``file://`` paths) under the
server's content-security policy.

The reference's ``ContentSecurityConfig`` (specs/openapi/inference/api.yaml:2890-2936): ``allowed_hosts`` whitelist,
``block_private_ips`` (default on: loopback, RFC 1918, link-local), ``max_download_size_bytes`` (100 MiB),
``download_timeout_seconds`` (30), ``max_image_dimension`` (2048: larger images are scaled down), ``allowed_paths``
prefixes for ``file://`` (and ``s3://``) URLs, ``user_agent`` ("AntflyDB/1.0").  Link downloads are off unless the
configuration allows them (``allow_downloads``); ``data:`` URLs always work.  Every redirect hop is checked against
the same rules, and the address a name resolves to is checked, not the name, so that a public name pointing at a
private address is refused as well.  ``s3://`` needs an object-store client, which this build does not carry.
"""
from __future__ import annotations

import base64
import ipaddress
import os
import socket
import urllib.error
import urllib.parse
import urllib.request
from dataclasses import dataclass, field
from typing import List, Optional, Tuple


class ContentError(ValueError):
    pass


@dataclass
class ContentSecurity:
    allow_downloads: bool = False
    allowed_hosts: List[str] = field(default_factory=list)
    block_private_ips: bool = True
    max_download_size_bytes: int = 100 * 1024 * 1024
    download_timeout_seconds: int = 30
    max_image_dimension: int = 2048
    allowed_paths: List[str] = field(default_factory=list)
    user_agent: str = "AntflyDB/1.0"

    @classmethod
    def from_dict(cls, d: Optional[dict], allow_downloads: bool = False) -> "ContentSecurity":
        d = dict(d or {})
        known = {k: d[k] for k in cls.__dataclass_fields__ if k in d and d[k] is not None}
        known.setdefault("allow_downloads", allow_downloads)
        out = cls(**known)
        if out.max_download_size_bytes < 0 or out.download_timeout_seconds < 1 or out.max_image_dimension < 1:
            raise ValueError("content_security: sizes and time-outs must be positive")
        return out


def _private(ip: str) -> bool:
    a = ipaddress.ip_address(ip)
    if getattr(a, "ipv4_mapped", None):
        a = a.ipv4_mapped
    return a.is_private or a.is_loopback or a.is_link_local or a.is_reserved or a.is_multicast or a.is_unspecified


class _NoRedirect(urllib.request.HTTPRedirectHandler):
    def redirect_request(self, req, fp, code, msg, headers, newurl):
        return None                                       # hops are followed by hand, each one checked


class ContentFetcher:
    def __init__(self, policy: Optional[ContentSecurity] = None, resolver=socket.getaddrinfo):
        self.policy = policy or ContentSecurity()
        self._resolve = resolver
        self._opener = urllib.request.build_opener(_NoRedirect)

    # -- checks --------------------------------------------------------------------------------------------
    def check_host(self, host: str) -> None:
        p = self.policy
        if p.allowed_hosts and host.lower() not in {h.lower() for h in p.allowed_hosts}:
            raise ContentError(f"host {host!r} is not in allowed_hosts")
        if not p.block_private_ips:
            return
        try:
            addrs = {ai[4][0] for ai in self._resolve(host, None)}
        except OSError as e:
            raise ContentError(f"cannot resolve {host!r}: {e}") from e
        for a in addrs:
            if _private(a):
                raise ContentError(f"host {host!r} resolves to the private address {a}")

    def check_path(self, path: str) -> str:
        real = os.path.realpath(path)
        allowed = self.policy.allowed_paths
        if allowed and not any(real == os.path.realpath(a).rstrip("/") or real.startswith(os.path.realpath(a).rstrip("/") + "/")
                               for a in allowed):
            raise ContentError(f"path {path!r} is outside allowed_paths")
        return real

    # -- fetch ---------------------------------------------------------------------------------------------
    def fetch(self, url: str) -> Tuple[bytes, str]:
        """-> (bytes, mime type or "")."""
        if not isinstance(url, str) or not url:
            raise ContentError("empty media reference")
        if url.startswith("data:"):
            if "," not in url:
                raise ContentError("malformed data: URL")
            head, payload = url.split(",", 1)
            mime = head[5:].split(";")[0].strip().lower()
            try:
                raw = base64.b64decode(payload, validate=True) if head.endswith(";base64") else \
                    urllib.parse.unquote_to_bytes(payload)
            except Exception as e:
                raise ContentError(f"data: URL is not valid base64: {e}") from e
            if self.policy.max_download_size_bytes and len(raw) > self.policy.max_download_size_bytes:
                raise ContentError("content exceeds max_download_size_bytes")
            return raw, mime
        scheme = urllib.parse.urlparse(url).scheme.lower()
        if scheme not in ("http", "https", "file", "s3"):
            raise ContentError("media must be a data: URL, an http(s):// link or a file:// path")
        if not self.policy.allow_downloads:
            raise ContentError("this server does not fetch links (allow_downloads is off); send a data: URL")
        if scheme == "s3":
            raise ContentError("s3:// links need an object-store client, which this build does not have")
        if scheme == "file":
            path = self.check_path(urllib.parse.unquote(urllib.parse.urlparse(url).path))
            size = os.path.getsize(path)
            if self.policy.max_download_size_bytes and size > self.policy.max_download_size_bytes:
                raise ContentError("content exceeds max_download_size_bytes")
            with open(path, "rb") as f:
                return f.read(), ""
        return self._http(url)

    def _http(self, url: str) -> Tuple[bytes, str]:
        p = self.policy
        for _hop in range(6):
            parts = urllib.parse.urlparse(url)
            if parts.scheme not in ("http", "https") or not parts.hostname:
                raise ContentError(f"redirect to an unsupported location {url!r}")
            self.check_host(parts.hostname)
            req = urllib.request.Request(url, headers={"User-Agent": p.user_agent or "AntflyDB/1.0"})
            try:
                resp = self._opener.open(req, timeout=p.download_timeout_seconds)
            except urllib.error.HTTPError as e:
                if e.code in (301, 302, 303, 307, 308) and e.headers.get("Location"):
                    url = urllib.parse.urljoin(url, e.headers["Location"])
                    continue
                raise ContentError(f"{url}: HTTP {e.code}") from e
            except (urllib.error.URLError, OSError) as e:
                raise ContentError(f"{url}: {getattr(e, 'reason', e)}") from e
            with resp:
                limit = p.max_download_size_bytes
                declared = resp.headers.get("Content-Length")
                if limit and declared and declared.isdigit() and int(declared) > limit:
                    raise ContentError("content exceeds max_download_size_bytes")
                chunks, got = [], 0
                while True:
                    buf = resp.read(1 << 20)
                    if not buf:
                        break
                    got += len(buf)
                    if limit and got > limit:
                        raise ContentError("content exceeds max_download_size_bytes")
                    chunks.append(buf)
                mime = (resp.headers.get("Content-Type") or "").split(";")[0].strip().lower()
                return b"".join(chunks), mime
        raise ContentError("too many redirects")

    # -- typed helpers -------------------------------------------------------------------------------------
    def image(self, url: str):
        """Decoded uint8 [H, W, 3] tensor; images larger than ``max_image_dimension`` on a side are scaled down."""
        from ..pipelines.multimodal import decode_image_bytes

        raw, _ = self.fetch(url)
        img = decode_image_bytes(raw)
        cap = self.policy.max_image_dimension
        h, w = int(img.shape[0]), int(img.shape[1])
        if cap and max(h, w) > cap:
            import torch

            s = cap / max(h, w)
            nh, nw = max(1, round(h * s)), max(1, round(w * s))
            t = img.permute(2, 0, 1)[None].float()
            t = torch.nn.functional.interpolate(t, size=(nh, nw), mode="bilinear", antialias=True, align_corners=False)
            img = t[0].permute(1, 2, 0).round().clamp(0, 255).to(img.dtype)
        return img
