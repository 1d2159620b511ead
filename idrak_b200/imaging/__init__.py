"""Imaging: Pillow-exact resampling, exact-coverage rasterisation of outlines and TrueType text, warps, blur and rank
filters, seeded scan / paper effects, page layout and file codecs - on CPU tensors and as CUDA kernels writing into
plain device buffers."""
from .codecs import ImageFormatError, decode, decode_bmp, decode_png, decode_pnm, encode, encode_bmp, encode_png, encode_pnm
from .effects import EFFECTS, PixelPass, apply, pixel_pass, random_pipeline
from .jpeg import decode_jpeg
from .font import FontError, TrueTypeFont, render_text
from .shaping import base_direction, layout_line, shape_arabic, visual_order
from .layout import Page, WordBox, compose_page, wrap
from .raster import Path, coverage_reference, ellipse, rasterize, rect, supersample_reference
from .resample import FILTERS, resize, taps
from .warp import (box_blur, gaussian_blur, max_filter, median_filter, min_filter, quad_to_quad, rank_filter, rotation, shear,
                   warp)
