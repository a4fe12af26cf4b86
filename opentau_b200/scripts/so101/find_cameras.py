"""``opentau-so101-find-cameras``: list the OpenCV capture devices that open."""

import json

from .devices import OpenCVCamera


def main(argv=None):
    print(json.dumps(OpenCVCamera.find_cameras(), indent=2))


if __name__ == "__main__":
    main()
