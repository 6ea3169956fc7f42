"""SM clock and throttle-reason sampling (nvidia-smi queries only; nothing is set) around a timed region."""
import statistics
import subprocess
import threading
import time


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self, wait_s: float = 5.0):
        """Starts nvidia-smi and waits for its first row, so that a short region is never left without samples."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "50"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
            return self
        t0 = time.perf_counter()
        while not self.rows and time.perf_counter() - t0 < wait_s and self.proc.poll() is None:
            time.sleep(0.01)
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.06)   # one more sampling period, so that the end of the region is covered
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, mx, reasons, power = [], None, set(), []
        for r in self.rows:
            if len(r) < 8:
                continue
            try:
                clocks.append(float(r[1]))
                mx = float(r[2])
                power.append(float(r[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # under load = the samples taken while the board drew at least half of the largest power seen
        loaded = [c for c, p in zip(clocks, power) if power and p >= 0.5 * max(power)] or clocks
        return {"sm_mhz": statistics.median(loaded) if loaded else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks), "power_w_max": max(power) if power else None}
