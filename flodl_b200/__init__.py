"""flodl_b200: a Blackwell-native deep-learning framework with floDl's API."""
