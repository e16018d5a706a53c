"""Process-wide logger: console plus ./amct_log/amct_pytorch.log.

Environment variables as in the reference (amct_pytorch/utils/log.py:33-36):
AMCT_LOG_LEVEL sets the console level, AMCT_LOG_FILE_LEVEL the file level
(debug/info/warning/error).  The log file is opened on the first message and a
read-only working directory only disables file logging.
"""
import logging
import os

_LEVELS = {'debug': logging.DEBUG, 'info': logging.INFO, 'warning': logging.WARNING, 'error': logging.ERROR}
LOG_DIR, LOG_FILE = 'amct_log', 'amct_pytorch.log'
_CHUNK = 500


def _level(env, default):
    return _LEVELS.get(os.environ.get(env, default).lower(), _LEVELS[default])


class _Logger:
    def __init__(self):
        self._log = logging.getLogger('amct_b200')
        self._log.setLevel(logging.DEBUG)
        self._log.propagate = False
        if not self._log.handlers:
            console = logging.StreamHandler()
            console.setLevel(_level('AMCT_LOG_LEVEL', 'info'))
            console.setFormatter(logging.Formatter('%(asctime)s - %(levelname)s - [AMCT]:%(message)s'))
            self._log.addHandler(console)
        self._file_ready = False

    def _ensure_file(self):
        if self._file_ready:
            return
        self._file_ready = True
        try:
            os.makedirs(LOG_DIR, mode=0o750, exist_ok=True)
            path = os.path.join(LOG_DIR, LOG_FILE)
            handler = logging.FileHandler(path)
            os.chmod(path, 0o640)
            handler.setLevel(_level('AMCT_LOG_FILE_LEVEL', 'info'))
            handler.setFormatter(logging.Formatter('%(asctime)s - %(levelname)s - [AMCT]:%(message)s'))
            self._log.addHandler(handler)
        except OSError:
            pass

    def _emit(self, fn, message, module):
        self._ensure_file()
        text = '[{}]: {}'.format(module, message)
        for i in range(0, len(text), _CHUNK):
            fn(text[i:i + _CHUNK])

    def logd(self, message, module='AMCT'):
        self._emit(self._log.debug, message, module)

    def logi(self, message, module='AMCT'):
        self._emit(self._log.info, message, module)

    def logw(self, message, module='AMCT'):
        self._emit(self._log.warning, message, module)

    def loge(self, message, module='AMCT'):
        self._emit(self._log.error, message, module)


LOGGER = _Logger()
