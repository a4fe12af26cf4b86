"""``opentau-so101-find-cameras``: list the OpenCV capture devices that open."""

import json

from .device_paths import stable_video_path
from .devices import OpenCVCamera


def main(argv=None):
    found = OpenCVCamera.find_cameras()
    for cam in found:
        idx = cam.get("index", cam.get("id"))
        node = idx if isinstance(idx, str) else (f"/dev/video{idx}" if idx is not None else None)
        cam["stable_path"] = stable_video_path(node)
    print(json.dumps(found, indent=2))


if __name__ == "__main__":
    main()
