"""Operational helpers around training runs: config diffs, log scraping, checkpoint summaries, filter-length checks.
Role of the reference's launcher/scripts/ directory (its S3 / wandb scrapers are tied to one site's buckets and
projects; the generic parts are restated here and work on local files)."""
