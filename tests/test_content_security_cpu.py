"""Media references under the content-security policy: data URLs, link downloads (off by default), host whitelist,
private-address blocking (also behind a redirect and behind a public-looking name), size and dimension limits,
file:// prefixes; and the endpoints using it."""
import base64
import http.server
import io
import threading

import pytest
import torch

from antfly_b200.api.content import ContentError, ContentFetcher, ContentSecurity


def _png(w=8, h=6, color=(200, 30, 30)):
    from PIL import Image

    buf = io.BytesIO()
    Image.new("RGB", (w, h), color).save(buf, "PNG")
    return buf.getvalue()


class _H(http.server.BaseHTTPRequestHandler):
    agents = []

    def log_message(self, *a):
        pass

    def do_GET(self):
        type(self).agents.append(self.headers.get("User-Agent"))
        if self.path == "/img.png":
            body = _png()
            self.send_response(200); self.send_header("Content-Type", "image/png")
            self.send_header("Content-Length", str(len(body))); self.end_headers(); self.wfile.write(body)
        elif self.path == "/big":
            self.send_response(200); self.send_header("Content-Type", "application/octet-stream"); self.end_headers()
            self.wfile.write(b"x" * 5000)
        elif self.path == "/hop":
            self.send_response(302); self.send_header("Location", "/img.png"); self.end_headers()
        elif self.path == "/away":
            self.send_response(302); self.send_header("Location", "http://10.1.2.3/secret"); self.end_headers()
        else:
            self.send_response(404); self.end_headers()


@pytest.fixture(scope="module")
def site():
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), _H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    yield f"http://127.0.0.1:{srv.server_address[1]}"
    srv.shutdown()
    srv.server_close()


def test_data_urls_and_the_default_policy(site):
    f = ContentFetcher()
    raw, mime = f.fetch("data:image/png;base64," + base64.b64encode(_png()).decode())
    assert mime == "image/png" and raw[:4] == b"\x89PNG"
    assert f.image("data:image/png;base64," + base64.b64encode(_png(10, 4)).decode()).shape == (4, 10, 3)
    for bad in (site + "/img.png", "file:///etc/hostname", "ftp://x/y", "", "data:image/png;base64"):
        with pytest.raises(ContentError):
            f.fetch(bad)
    with pytest.raises(ContentError, match="base64"):
        f.fetch("data:image/png;base64,@@@")
    with pytest.raises(ValueError):
        ContentSecurity.from_dict({"download_timeout_seconds": 0})


def test_link_downloads_hosts_private_addresses_and_limits(site, tmp_path):
    # downloads on, but the loopback address is private: refused until the operator says otherwise
    strict = ContentFetcher(ContentSecurity(allow_downloads=True))
    with pytest.raises(ContentError, match="private"):
        strict.fetch(site + "/img.png")
    # a public-looking name that resolves to a private address is refused as well
    fake_dns = lambda host, port: [(2, 1, 6, "", ("192.168.1.7", 0))]
    with pytest.raises(ContentError, match="private"):
        ContentFetcher(ContentSecurity(allow_downloads=True), resolver=fake_dns).check_host("cdn.example.com")
    open_ = ContentFetcher(ContentSecurity(allow_downloads=True, block_private_ips=False, allowed_hosts=["127.0.0.1"],
                                           user_agent="probe/1"))
    raw, mime = open_.fetch(site + "/img.png")
    assert raw == _png() and mime == "image/png" and "probe/1" in _H.agents
    assert open_.fetch(site + "/hop")[0] == _png()                       # a redirect inside the allowed host
    with pytest.raises(ContentError, match="allowed_hosts"):             # a redirect that leaves it
        open_.fetch(site + "/away")
    with pytest.raises(ContentError, match="404"):
        open_.fetch(site + "/nothing")
    with pytest.raises(ContentError, match="allowed_hosts"):
        ContentFetcher(ContentSecurity(allow_downloads=True, block_private_ips=False, allowed_hosts=["example.com"])
                       ).fetch(site + "/img.png")
    small = ContentFetcher(ContentSecurity(allow_downloads=True, block_private_ips=False, max_download_size_bytes=1000))
    with pytest.raises(ContentError, match="max_download_size_bytes"):
        small.fetch(site + "/big")
    # blocked behind a redirect too when private addresses are blocked
    hop = ContentFetcher(ContentSecurity(allow_downloads=True, block_private_ips=False))
    with pytest.raises(ContentError):
        ContentFetcher(ContentSecurity(allow_downloads=True, block_private_ips=True,
                                       allowed_hosts=[]), resolver=lambda h, p: [(2, 1, 6, "", ("93.184.216.34" if h == "127.0.0.1" else "10.1.2.3", 0))]
                       ).fetch(site + "/away")
    # files: prefix whitelist, symlinks resolved
    (tmp_path / "ok").mkdir()
    (tmp_path / "ok" / "a.png").write_bytes(_png())
    (tmp_path / "secret.png").write_bytes(_png())
    (tmp_path / "ok" / "link.png").symlink_to(tmp_path / "secret.png")
    files = ContentFetcher(ContentSecurity(allow_downloads=True, allowed_paths=[str(tmp_path / "ok")]))
    assert files.fetch(f"file://{tmp_path}/ok/a.png")[0] == _png()
    for bad in (f"file://{tmp_path}/secret.png", f"file://{tmp_path}/ok/link.png", f"file://{tmp_path}/ok/../secret.png"):
        with pytest.raises(ContentError, match="allowed_paths"):
            files.fetch(bad)
    with pytest.raises(ContentError, match="object-store"):
        files.fetch("s3://bucket/key.png")
    # oversized images are scaled down, keeping the aspect ratio
    big = "data:image/png;base64," + base64.b64encode(_png(400, 100)).decode()
    img = ContentFetcher(ContentSecurity(max_image_dimension=100)).image(big)
    assert img.shape == (25, 100, 3) and img.dtype == torch.uint8 and int(img[..., 0].float().mean()) in range(195, 205)


def test_endpoints_apply_the_policy(site):
    from fastapi.testclient import TestClient

    from antfly_b200.api.model_manager import ModelManager
    from antfly_b200.api.server import create_app

    mgr = ModelManager(models_dir="/nonexistent", device="cpu")
    mgr.register_random("random:tiny", "embedder")
    body = {"model": "random:tiny", "input": [{"type": "image_url", "image_url": {"url": site + "/img.png"}}]}
    r = TestClient(create_app(mgr)).post("/ai/v1/embed", json=body)
    assert r.status_code == 400 and "allow_downloads" in r.text
    assert TestClient(create_app(mgr)).get("/ai/v1/models").json()["allow_downloads"] is False
    app = create_app(mgr, content_security={"allow_downloads": True, "block_private_ips": False})
    c = TestClient(app)
    assert c.get("/ai/v1/models").json()["allow_downloads"] is True
    r = c.post("/ai/v1/embed", json=body)
    # the link is fetched now; the byte-level test model has no image tower, which is what the reply says
    assert r.status_code == 400 and "image" in r.text and "allow_downloads" not in r.text
