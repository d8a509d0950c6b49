"""The HTTP report server serves the live series (CPU)."""
import json
import urllib.request

from rembrandt_b200.utils.report import ReportServer


def test_report_server_serves_page_and_series():
    srv = ReportServer(port=0)
    try:
        srv.update_training(10, 2.5, 0.1)
        srv.update_training(20, 1.5, 0.4)
        srv.update_validation(20, 1.7, 0.35)
        base = f"http://127.0.0.1:{srv.port}"
        page = urllib.request.urlopen(base + "/", timeout=5).read().decode()
        assert "<canvas" in page
        data = json.loads(urllib.request.urlopen(base + "/api/v0/train_loss.json", timeout=5).read())
        assert data["train_loss"] == [[10, 2.5], [20, 1.5]] and data["valid_accuracy"] == [[20, 0.35]]
    finally:
        srv.close()
