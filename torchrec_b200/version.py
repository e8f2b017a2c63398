"""Package version.  ``api_level`` is the release line of the recommendation-library API surface this package follows."""
__version__ = "0.1.0"
api_level = "1.4"
git_version = "Unknown"
