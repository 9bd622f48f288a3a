"""``get_file`` with hash validation and guarded archive extraction, plus path helpers
(keras/src/utils/file_utils.py)."""

import hashlib
import os
import re
import shutil
import tarfile
import urllib.error
import urllib.parse
import urllib.request
import zipfile

from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.utils import io_utils
from keras_b200.utils.progbar import Progbar


def path_to_string(path):
    if isinstance(path, os.PathLike):
        return os.fspath(path)
    return path


def resolve_path(path):
    return os.path.realpath(os.path.abspath(path))


def is_path_in_dir(path, base_dir):
    return resolve_path(os.path.join(base_dir, path)).startswith(base_dir)


def is_link_in_dir(info, base):
    tip = resolve_path(os.path.join(base, os.path.dirname(info.name)))
    return is_path_in_dir(info.linkname, base_dir=tip)


def filter_safe_zipinfos(members):
    base_dir = resolve_path(".")
    for finfo in members:
        valid = True
        if not is_path_in_dir(finfo.filename, base_dir):
            valid = False
            import warnings

            warnings.warn(f"Skipping invalid path during archive extraction: '{finfo.filename}'.", stacklevel=2)
        if valid:
            yield finfo


def filter_safe_tarinfos(members):
    base_dir = resolve_path(".")
    for finfo in members:
        valid = True
        if finfo.issym() or finfo.islnk():
            if not is_link_in_dir(finfo, base_dir):
                valid = False
        elif not is_path_in_dir(finfo.name, base_dir):
            valid = False
        if not valid:
            import warnings

            warnings.warn(f"Skipping invalid path during archive extraction: '{finfo.name}'.", stacklevel=2)
        else:
            yield finfo


def extract_open_archive(archive, path="."):
    """Extract an open zip or tar archive, skipping members that would land outside ``path``."""
    cwd = os.getcwd()
    os.makedirs(path, exist_ok=True)
    os.chdir(path)
    try:
        if isinstance(archive, zipfile.ZipFile):
            archive.extractall(".", members=filter_safe_zipinfos(archive.infolist()))
        else:
            kwargs = {"filter": "data"} if hasattr(tarfile, "data_filter") else {}
            archive.extractall(".", members=filter_safe_tarinfos(archive), **kwargs)
    finally:
        os.chdir(cwd)


def extract_archive(file_path, path=".", archive_format="auto"):
    if archive_format is None:
        return False
    if archive_format == "auto":
        archive_format = ["tar", "zip"]
    if isinstance(archive_format, str):
        archive_format = [archive_format]
    file_path = path_to_string(file_path)
    path = path_to_string(path)
    for archive_type in archive_format:
        if archive_type == "tar":
            open_fn, is_match_fn = tarfile.open, tarfile.is_tarfile
        elif archive_type == "zip":
            open_fn, is_match_fn = zipfile.ZipFile, zipfile.is_zipfile
        else:
            raise NotImplementedError(archive_type)
        if is_match_fn(file_path):
            with open_fn(file_path) as archive:
                try:
                    extract_open_archive(archive, path)
                except (tarfile.TarError, RuntimeError, KeyboardInterrupt):
                    if os.path.exists(path):
                        if os.path.isfile(path):
                            os.remove(path)
                        else:
                            shutil.rmtree(path)
                    raise
            return True
    return False


def resolve_hasher(algorithm, file_hash=None):
    if algorithm == "sha256":
        return hashlib.sha256()
    if algorithm == "auto" and file_hash is not None and len(file_hash) == 64:
        return hashlib.sha256()
    return hashlib.md5()


def hash_file(fpath, algorithm="sha256", chunk_size=65535):
    hasher = resolve_hasher(algorithm) if isinstance(algorithm, str) else algorithm
    with open(fpath, "rb") as f:
        for chunk in iter(lambda: f.read(chunk_size), b""):
            hasher.update(chunk)
    return hasher.hexdigest()


def validate_file(fpath, file_hash, algorithm="auto", chunk_size=65535):
    hasher = resolve_hasher(algorithm, file_hash)
    return str(hash_file(fpath, hasher, chunk_size)) == str(file_hash)


@keras_export("keras.utils.get_file")
def get_file(fname=None, origin=None, untar=False, md5_hash=None, file_hash=None, cache_subdir="datasets", hash_algorithm="auto", extract=False,
             archive_format="auto", cache_dir=None, force_download=False):
    """Download ``origin`` into the cache (``~/.keras/<cache_subdir>``) unless a valid copy is already there."""
    if origin is None:
        raise ValueError('Please specify the "origin" argument (URL of the file to download).')
    if cache_dir is None:
        cache_dir = config.keras_home()
    if md5_hash is not None and file_hash is None:
        file_hash = md5_hash
        hash_algorithm = "md5"
    datadir_base = os.path.expanduser(cache_dir)
    if not os.access(datadir_base, os.W_OK):
        datadir_base = os.path.join("/tmp", ".keras")
    datadir = os.path.join(datadir_base, cache_subdir)
    os.makedirs(datadir, exist_ok=True)
    fname = path_to_string(fname)
    if not fname:
        fname = os.path.basename(urllib.parse.urlsplit(origin).path)
        if not fname:
            raise ValueError(f"Can't parse the file name from the origin provided: '{origin}'.Please specify the `fname` argument.")
    elif os.sep in fname:
        raise ValueError(f"Paths are no longer accepted as the `fname` argument. To specify the file's parent directory, use the `cache_dir` argument. Received: fname={fname}")
    if extract or untar:
        if untar:
            archive_format = "tar"
        fname_no_ext = fname
        for ext in (".tar.gz", ".tar.bz2", ".tar", ".zip", ".tgz"):
            if fname_no_ext.endswith(ext):
                fname_no_ext = fname_no_ext[: -len(ext)]
                break
        download_target = os.path.join(datadir, fname)
        extraction_dir = os.path.join(datadir, fname_no_ext + "_extracted") if fname_no_ext == fname else os.path.join(datadir, fname_no_ext)
        if fname_no_ext == fname:
            pass
    else:
        download_target = os.path.join(datadir, fname)
        extraction_dir = None
    download = force_download
    if not force_download:
        if os.path.exists(download_target):
            if file_hash is not None and not validate_file(download_target, file_hash, algorithm=hash_algorithm):
                io_utils.print_msg(f"A local file was found, but it seems to be incomplete or outdated because the {hash_algorithm} file hash does not match the original value of {file_hash} so we will re-download the data.")
                download = True
        else:
            download = True
    if download:
        io_utils.print_msg(f"Downloading data from {origin}")

        class DLProgbar:
            def __init__(self):
                self.progbar = None
                self.finished = False

            def __call__(self, block_num, block_size, total_size):
                if total_size == -1:
                    total_size = None
                if not self.progbar:
                    self.progbar = Progbar(total_size)
                current = block_num * block_size
                if total_size is None:
                    self.progbar.update(current)
                elif current < total_size:
                    self.progbar.update(current)
                elif not self.finished:
                    self.progbar.update(self.progbar.target)
                    self.finished = True

        error_msg = "URL fetch failure on {}: {} -- {}"
        try:
            try:
                urllib.request.urlretrieve(origin, download_target, DLProgbar())
            except urllib.error.HTTPError as e:
                raise Exception(error_msg.format(origin, e.code, e.msg))
            except urllib.error.URLError as e:
                raise Exception(error_msg.format(origin, e.errno, e.reason))
        except (Exception, KeyboardInterrupt):
            if os.path.exists(download_target):
                os.remove(download_target)
            raise
        if os.path.exists(download_target) and file_hash is not None and not validate_file(download_target, file_hash, algorithm=hash_algorithm):
            raise ValueError(f"Incomplete or corrupted file detected. The {hash_algorithm} file hash does not match the provided value of {file_hash}.")
    if extract or untar:
        status = extract_archive(download_target, extraction_dir, archive_format)
        if not status:
            import warnings

            warnings.warn("Could not extract archive.", stacklevel=2)
        return extraction_dir
    return download_target


def exists(path):
    return os.path.exists(path)


def File(path, mode="r"):
    return open(path, mode)


def join(path, *paths):
    return os.path.join(path, *paths)


def isdir(path):
    return os.path.isdir(path)


def remove(path):
    return os.remove(path)


def rmtree(path):
    return shutil.rmtree(path)


def listdir(path):
    return os.listdir(path)


def copy(src, dst):
    return shutil.copy(src, dst)


def makedirs(path):
    return os.makedirs(path, exist_ok=True)


def is_remote_path(filepath):
    return bool(re.match(r"^(/cns|/cfs|/gcs|/hdfs|/readahead|/placer|/tfhub|.*://).*$", str(filepath)))
