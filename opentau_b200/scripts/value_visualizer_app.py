"""Interactive value-function viewer: timeline scrubber, camera frame and value curve of one episode.

The reference app (``src/opentau/scripts/value_visualizer_app.py:50-347``) is a Streamlit page: a slider over the frames
of one episode, the camera image at the slider, the value curve with a marker at the current step, a smoothing window,
and three summary figures (mean / final value, steps).  This one serves the same page from the standard library's HTTP
server, so it needs no GUI toolkit on the training box: the browser draws the curve on a canvas and fetches
``/frame/<i>.jpg`` as the slider moves.

    python -m opentau_b200.scripts.value_visualizer_app --dataset-config dataset_config.json --values values.json \\
        [--episode 0] [--port 8501]

``dataset_config.json`` is ``{"datasets": [{"root": ..., "repo_id": ..., "episodes": [...]}]}``; a plain
``--dataset-root`` works too.  Value files: both layouts that ``value_visualizer.load_values`` reads.
"""

from __future__ import annotations

import argparse
import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from pathlib import Path

import numpy as np

from .value_visualizer import episode_frames, load_values

PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>Value function viewer</title>
<style>body{font-family:sans-serif;margin:16px}#wrap{display:flex;gap:24px}#cam{width:448px;border:1px solid #ccc}
.m{display:inline-block;margin-right:32px}.m b{font-size:22px;display:block}</style></head><body>
<h2>Value function analysis &mdash; episode <span id="ep"></span></h2>
<div id="wrap"><div><h3>Camera (step <span id="step">0</span>)</h3><img id="cam"/>
<p>Predicted value <b id="val"></b><br/><small id="cap"></small></p></div>
<div><h3>Value function V(s)</h3><canvas id="cv" width="720" height="360"></canvas><br/>
<input id="sl" type="range" min="0" max="0" value="0" style="width:720px"/><br/>
<label>smoothing window <input id="sm" type="number" min="1" max="10" value="3"/></label></div></div><hr/>
<div><span class="m">mean value<b id="mean"></b></span><span class="m">final value<b id="final"></b></span>
<span class="m">steps<b id="n"></b></span></div>
<script>
let D=null;const $=id=>document.getElementById(id);
function smooth(v,w){return v.map((_,i)=>{let a=Math.max(0,i-w+1),s=0;for(let j=a;j<=i;j++)s+=v[j];return s/(i-a+1)})}
function draw(){const c=$("cv"),g=c.getContext("2d"),v=smooth(D.value,+$("sm").value),n=v.length,i=+$("sl").value;
 const lo=Math.min(...v),hi=Math.max(...v)>lo?Math.max(...v):lo+1;const X=k=>40+k/Math.max(n-1,1)*(c.width-60),
 Y=y=>c.height-30-(y-lo)/(hi-lo)*(c.height-50);g.clearRect(0,0,c.width,c.height);g.strokeStyle="#ccc";
 g.strokeRect(0,0,c.width,c.height);g.fillText(hi.toFixed(3),4,Y(hi)+4);g.fillText(lo.toFixed(3),4,Y(lo)+4);
 g.beginPath();g.strokeStyle="#1f77b4";v.forEach((y,k)=>k?g.lineTo(X(k),Y(y)):g.moveTo(X(k),Y(y)));g.stroke();
 g.beginPath();g.strokeStyle="#d62728";g.moveTo(X(i),10);g.lineTo(X(i),c.height-30);g.stroke();
 g.beginPath();g.fillStyle="#d62728";g.arc(X(i),Y(v[i]),4,0,7);g.fill();g.fillStyle="#000";
 $("step").textContent=i;$("val").textContent=D.value[i].toFixed(3);
 $("cap").textContent="episode "+D.episode+", t = "+D.t[i].toFixed(2)+" s";$("cam").src="/frame/"+D.frame[i]+".jpg"}
fetch("/api/episode").then(r=>r.json()).then(d=>{D=d;$("ep").textContent=d.episode;$("sl").max=d.value.length-1;
 $("mean").textContent=d.mean.toFixed(3);$("final").textContent=d.final.toFixed(3);$("n").textContent=d.value.length;
 $("sl").oninput=draw;$("sm").oninput=draw;draw()});
</script></body></html>"""


def load_dataset_config(path: str | Path) -> tuple[Path, str, list[int]]:
    """``dataset_config.json`` -> (root, repo id, episode indices) of its first dataset."""
    cfg = json.loads(Path(path).read_text())
    datasets = cfg.get("datasets", [])
    if not datasets:
        raise ValueError(f"no 'datasets' in {path}")
    first = datasets[0]
    eps = first.get("episodes", [0])
    eps = sorted(eps) if isinstance(eps, list) else list(range(int(eps)))
    return Path(first["root"]).resolve(), first.get("repo_id", "local/dataset"), eps


def episode_payload(values: dict[int, list[dict]], episode: int, fps: float | None) -> dict:
    """What the page needs for one episode: time, value and the dataset frame index of every value."""
    if episode not in values:
        raise KeyError(f"episode {episode} not in the value file (has {sorted(values)[:8]}...)")
    rows = values[episode]
    t = [float(r["t"]) for r in rows]
    v = [float(r["value"]) for r in rows]
    frame = [int(round(x * fps)) if fps else int(round(x)) for x in t]
    finite = [x for x in v if np.isfinite(x)]
    return {"episode": episode, "t": t, "value": v, "frame": frame,
            "mean": float(np.mean(finite)) if finite else 0.0, "final": v[-1] if v else 0.0}


class ViewerState:
    """Episode data plus a small cache of encoded camera frames (the slider revisits neighbours)."""

    def __init__(self, values: dict[int, list[dict]], episode: int, dataset_root: Path | None, fps: float | None,
                 max_side: int = 448):
        self.root, self.episode, self.max_side = dataset_root, episode, max_side
        self.payload = episode_payload(values, episode, fps)
        self._jpeg: dict[int, bytes] = {}
        self._lock = threading.Lock()

    def frame_jpeg(self, index: int) -> bytes | None:
        import cv2
        with self._lock:
            if index in self._jpeg:
                return self._jpeg[index]
        if self.root is None:
            return None
        got = episode_frames(self.root, self.episode, 1, indices=[index])
        if not got:
            return None
        img = got[0][1]
        s = self.max_side / max(img.shape[:2])
        if s < 1:
            img = cv2.resize(img, (round(img.shape[1] * s), round(img.shape[0] * s)), interpolation=cv2.INTER_AREA)
        ok, buf = cv2.imencode(".jpg", np.ascontiguousarray(img[:, :, ::-1]))
        if not ok:
            return None
        with self._lock:
            if len(self._jpeg) > 512:
                self._jpeg.clear()
            self._jpeg[index] = buf.tobytes()
        return self._jpeg[index]


def make_server(state: ViewerState, host: str = "127.0.0.1", port: int = 8501) -> ThreadingHTTPServer:
    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *a):  # quiet
            pass

        def _send(self, code: int, ctype: str, body: bytes) -> None:
            self.send_response(code)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):  # noqa: N802 - http.server API
            path = self.path.split("?", 1)[0]
            if path in ("/", "/index.html"):
                return self._send(200, "text/html; charset=utf-8", PAGE.encode())
            if path == "/api/episode":
                return self._send(200, "application/json", json.dumps(state.payload).encode())
            if path.startswith("/frame/") and path.endswith(".jpg"):
                try:
                    data = state.frame_jpeg(int(path[len("/frame/"):-4]))
                except ValueError:
                    data = None
                if data is None:
                    return self._send(404, "text/plain", b"no image for this frame")
                return self._send(200, "image/jpeg", data)
            return self._send(404, "text/plain", b"not found")

    return ThreadingHTTPServer((host, port), Handler)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--values", required=True)
    ap.add_argument("--dataset-config", default=None)
    ap.add_argument("--dataset-root", default=None)
    ap.add_argument("--episode", type=int, default=None)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8501)
    a = ap.parse_args(argv)
    root, episodes = (Path(a.dataset_root) if a.dataset_root else None), None
    if a.dataset_config:
        root, _, episodes = load_dataset_config(a.dataset_config)
    fps = None
    if root is not None:
        from ..datasets.utils import load_info
        fps = float(load_info(root)["fps"])
    raw = json.loads(Path(a.values).read_text())
    per_frame = any(isinstance(v, list) for v in raw.values())          # frame-indexed file: seconds need the fps
    values = load_values(a.values, fps if per_frame else None)
    episode = a.episode if a.episode is not None else (episodes[0] if episodes else sorted(values)[0])
    server = make_server(ViewerState(values, episode, root, fps), a.host, a.port)
    print(f"serving episode {episode} on http://{a.host}:{server.server_address[1]}/")
    try:
        server.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        server.server_close()


if __name__ == "__main__":
    main()
