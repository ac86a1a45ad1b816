// Command-line front end: parse, list devices or run every selected backend with
// the text logger, then write the requested result files once at the end
// (the flow of the reference's src/cli/main.cpp:151-211).
#include <iostream>

#include <common/logger_text.h>
#include <common/options.h>

#include "backend_table.hpp"

int main(int argc, char **argv)
{
    CliOptions opts;
    parseCliOptions(argc, argv, opts);
    clpeak::setVerbose(opts.verbose);

    if (opts.listDevices) {
        for (const auto &b : clpeakBackends())
            if (!(opts.*(b.skip)))
                b.printInventory(b.enumerate(), std::cout);
        return 0;
    }

    ResultStore rows;
    DeviceInfoStore devices;
    int status = 0, ran = 0;
    for (const auto &b : clpeakBackends()) {
        if (opts.*(b.skip))
            continue;
        ++ran;
        std::unique_ptr<Peak> peak = b.create();
        peak->log.reset(new LoggerText(std::cout, opts.compareFile, opts.describe));
        peak->applyOptions(opts);
        status |= peak->runAll();
        rows.insert(rows.end(), peak->log->results.begin(), peak->log->results.end());
        devices.insert(devices.end(), peak->log->devices.begin(), peak->log->devices.end());
    }
    if (opts.namedAbsentBackend) {
        std::cerr << "clpeak: the native CPU backend is not built into this binary (CUDA backend only)\n";
        if (ran == 0)
            status |= 1;
    }
    if (opts.enableJson && !saveJson(rows, opts.jsonFile, devices)) status |= 1;
    if (opts.enableCsv && !saveCsv(rows, opts.csvFile)) status |= 1;
    if (opts.enableXml && !saveXml(rows, opts.xmlFile, devices)) status |= 1;
    return status;
}
