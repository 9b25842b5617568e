"""Feature-compute functions with the reference's names and argument order
(spira/nn/functional/convolution.py:14-174)."""
__all__ = ['cuda_time_gather', 'cuda_time_scatter', 'sparse_convolution_forward_ws', 'sparse_convolution_forward_ws_merged',
           'sparse_convolution_forward_os', 'sparse_convolution_forward_hs', 'sparse_convolution_forward_hs_merged',
           'cuda_time_gemm', 'set_gemm_parallel_level']

from typing import Optional

import torch

from spira_b200.nn.functional import _C

GEMM_PARALLEL_LEVEL = 4


def set_gemm_parallel_level(level: int):
    global GEMM_PARALLEL_LEVEL
    GEMM_PARALLEL_LEVEL = level


def cuda_time_gather(weights, source_masks, target_masks, kernel_map_sizes, tile_size: int, is_hybrid: bool = False,
                     threshold: float = 0) -> float:
    return _C.cuda_time_gather(tile_size, threshold, is_hybrid, weights, source_masks, target_masks, kernel_map_sizes)


def cuda_time_scatter(weights, source_masks, target_masks, kernel_map_sizes, tile_size: int, is_hybrid: bool = False,
                      threshold: float = 0):
    return _C.cuda_time_scatter(tile_size, threshold, is_hybrid, weights, source_masks, target_masks, kernel_map_sizes)


def cuda_time_gemm(weights, source_masks, target_masks, kernel_map_sizes, parallel: Optional[int] = None,
                   is_hybrid: bool = False, threshold: float = 0):
    if parallel is None:
        parallel = GEMM_PARALLEL_LEVEL
    return _C.cuda_time_gemm(parallel, threshold, is_hybrid, weights, source_masks, target_masks, kernel_map_sizes)


def sparse_convolution_forward_ws(num_sources: int, num_targets: int, sources, weights, source_masks, target_masks,
                                  kernel_map_sizes, gather_tile_size: int, scatter_tile_size: int,
                                  parallel: Optional[int] = None, threshold: Optional[float] = 0) -> torch.Tensor:
    if sources.is_cuda:
        if parallel is None:
            parallel = GEMM_PARALLEL_LEVEL
        return _C.cuda_sparse_convolution_forward_ws(num_sources, num_targets, gather_tile_size, scatter_tile_size, parallel,
                                                     threshold, sources.contiguous(), weights.contiguous(), source_masks,
                                                     target_masks, kernel_map_sizes)
    raise NotImplementedError


def sparse_convolution_forward_ws_merged(num_sources: int, num_targets: int, sources, weights, naddrs, qnaddrs, nbmaps,
                                         mapsize: int, qmapsize: int, transpose: Optional[bool] = False) -> torch.Tensor:
    if sources.is_cuda:
        return _C.cuda_sparse_convolution_forward_ws_merged(num_sources, num_targets, sources.contiguous(), weights.contiguous(),
                                                            naddrs.contiguous(), qnaddrs.contiguous(), nbmaps.contiguous(),
                                                            mapsize, qmapsize, transpose)
    raise NotImplementedError


def sparse_convolution_forward_hs(num_sources: int, num_targets: int, sources, weights, source_masks, target_masks,
                                  kernel_map_sizes, out_in_map, gather_tile_size: int, scatter_tile_size: int,
                                  parallel: Optional[int] = None, threshold: Optional[float] = 0) -> torch.Tensor:
    if sources.is_cuda:
        if parallel is None:
            parallel = GEMM_PARALLEL_LEVEL
        return _C.cuda_sparse_convolution_forward_hs(num_sources, num_targets, gather_tile_size, scatter_tile_size, parallel,
                                                     threshold, sources.contiguous(), weights.contiguous(), source_masks,
                                                     target_masks, kernel_map_sizes, out_in_map)
    raise NotImplementedError


def sparse_convolution_forward_hs_merged(num_sources: int, num_targets: int, sources, weights, naddrs, qnaddrs, nbmaps,
                                         out_in_map, mapsize: int, qmapsize: int,
                                         transpose: Optional[bool] = False) -> torch.Tensor:
    if sources.is_cuda:
        return _C.cuda_sparse_convolution_forward_hs_merged(num_sources, num_targets, sources.contiguous(), weights.contiguous(),
                                                            naddrs.contiguous(), qnaddrs.contiguous(), nbmaps.contiguous(),
                                                            out_in_map, mapsize, qmapsize, transpose)
    raise NotImplementedError


def sparse_convolution_forward_os(num_sources: int, num_targets: int, out_in_map, sources, weights) -> torch.Tensor:
    if sources.is_cuda:
        return _C.cuda_sparse_convolution_forward_os(num_sources, num_targets, out_in_map.contiguous(), sources.contiguous(),
                                                     weights.contiguous())
    raise NotImplementedError
