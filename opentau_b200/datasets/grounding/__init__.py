from .loc_codec import (loc_tokens_to_points, loc_tokens_to_xyxy, points_to_loc_tokens, xyxy_to_loc_tokens)

__all__ = ["xyxy_to_loc_tokens", "points_to_loc_tokens", "loc_tokens_to_xyxy", "loc_tokens_to_points"]
